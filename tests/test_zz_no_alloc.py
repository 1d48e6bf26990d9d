"""The allocation-free index build (s3r_build_key_csr_static) against the regular entry point.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  Some hosts of the library cannot allocate device memory at the point of the call (all of it
was given to another runtime at start-up, or a synchronising cudaMalloc is not acceptable there);
for them the scratch of the index build sits in a fixed buffer inside the library.  The results
must be identical to the caller-workspace entry point, call after call, although the buffer keeps
the previous call's contents."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _table(seed, B, H, Nq, K, Nkb):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, Nkb, (B, H, Nq, K), generator=g, dtype=torch.int32)
    idx[:, :, 0, 0] = -1                       # dropped
    idx[:, :, 1, 1] = Nkb + 2                  # out of range: dropped
    idx[:, :, 2, :] = 3                        # one query block listing a key block K times
    return idx.to(DEV)


def _regular(lib, idx, Nkb):
    from speed3r_b200 import _lib
    B, H, Nq, K = idx.shape
    offsets = torch.empty(B, H, Nkb + 1, device=DEV, dtype=torch.int32)
    qids = torch.full((B, H, Nq * K), -1, device=DEV, dtype=torch.int32)
    n = lib.s3r_csr_workspace_bytes(B, H, Nq, K, Nkb)
    ws = torch.empty(n, device=DEV, dtype=torch.uint8)
    _lib.check(lib.s3r_build_key_csr(idx.data_ptr(), offsets.data_ptr(), qids.data_ptr(), B, H, Nq, K, Nkb,
                                     ws.data_ptr(), n, torch.cuda.current_stream().cuda_stream), "s3r_build_key_csr")
    return offsets, qids


def _static(lib, idx, Nkb):
    from speed3r_b200 import _lib
    B, H, Nq, K = idx.shape
    offsets = torch.empty(B, H, Nkb + 1, device=DEV, dtype=torch.int32)
    qids = torch.full((B, H, Nq * K), -1, device=DEV, dtype=torch.int32)
    _lib.check(lib.s3r_build_key_csr_static(idx.data_ptr(), offsets.data_ptr(), qids.data_ptr(), B, H, Nq, K, Nkb,
                                            torch.cuda.current_stream().cuda_stream), "s3r_build_key_csr_static")
    return offsets, qids


def test_static_scratch_matches_workspace_entry_point_twice(lib):
    # two different tables back to back: the second call finds the first call's leftovers in the buffer
    for seed, shape in ((1, (2, 16, 384, 32, 384)), (2, (1, 4, 100, 16, 130))):
        B, H, Nq, K, Nkb = shape
        idx = _table(seed, B, H, Nq, K, Nkb)
        off_a, q_a = _regular(lib, idx, Nkb)
        off_b, q_b = _static(lib, idx, Nkb)
        torch.cuda.synchronize()
        assert torch.equal(off_a, off_b), "offsets differ between the two entry points"
        assert torch.equal(q_a, q_b), "query-block lists differ between the two entry points"
        # and the result is a correct CSR: ascending query ids inside every key block's segment
        off = off_b.cpu()
        q = q_b.cpu()
        for n in (0, 3, Nkb - 1):
            seg = q[0, 0, off[0, 0, n]:off[0, 0, n + 1]]
            assert (seg[1:] >= seg[:-1]).all()
        assert int(off[0, 0, 4] - off[0, 0, 3]) >= K         # block 3 was listed K times by query block 2


def test_static_scratch_refuses_tables_beyond_its_buffer(lib):
    from speed3r_b200 import _lib
    B, H, Nq, K, Nkb = 1, 16, 63000, 32, 63000              # 1000 views: needs ~133 MB of scratch
    assert lib.s3r_csr_workspace_bytes(B, H, Nq, K, Nkb) > (8 << 20)
    dummy = torch.zeros(64, device=DEV, dtype=torch.int32)
    rc = lib.s3r_build_key_csr_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), B, H, Nq, K, Nkb, None)
    assert rc == -6 and "built-in buffer" in _lib.last_error()
