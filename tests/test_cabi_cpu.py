"""CPU-side checks of the C-ABI boundary: the library loads, exports every function the header
declares, and rejects bad arguments before touching the GPU (no compute is launched here)."""
import ctypes as C
import os
import re

import pytest
import torch

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "speed3r_b200.h")
CHECK_HEADER = os.path.join(ROOT, "include", "speed3r_b200_check.h")


def declared_functions(header=HEADER):
    src = open(header).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(s3r_[a-z0-9_]+)\s*\(", src)))


def test_header_and_binding_list_agree():
    from speed3r_b200 import _lib
    assert declared_functions() == sorted(_lib.SIGNATURES)
    assert declared_functions(CHECK_HEADER) == sorted(_lib.CHECK_SIGNATURES)


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but missing from the library"
    assert lib.s3r_version() >= 100
    assert not hasattr(lib, "s3r_check_sel_attn_fwd"), "tests-only kernels must not ship in the product library"


def test_check_library_exports_every_declared_symbol():
    from speed3r_b200 import _lib
    chk = _lib.load_check()
    for name in declared_functions(CHECK_HEADER):
        assert hasattr(chk, name), f"{name} is declared in the check header but missing from the check library"
    import ctypes
    assert chk.s3r_check_wait_gives_up(0, None, None) == -4          # argument errors need no GPU


def test_argument_errors_are_reported_without_a_gpu(lib):
    from speed3r_b200 import _lib
    # NULL pointers
    rc = lib.s3r_pool_fwd(None, 0, 0, 0, None, 1, 1, 16, 64, 16, 16, None)
    assert rc == -4 and "NULL" in _lib.last_error()
    buf = (C.c_uint16 * 4096)()
    p = C.addressof(buf)
    p = (p + 255) & ~255
    # head_dim not a multiple of 8
    rc = lib.s3r_pool_fwd(p, 0, 0, 8, p, 1, 1, 16, 60, 16, 16, None)
    assert rc == -2
    # sequence shorter than the pooling window
    rc = lib.s3r_pool_fwd(p, 0, 0, 64, p, 1, 1, 8, 64, 16, 16, None)
    assert rc == -1
    # misaligned pointer
    rc = lib.s3r_pool_fwd(p + 2, 0, 0, 64, p, 1, 1, 16, 64, 16, 16, None)
    assert rc == -3
    # unsupported head_dim / top-k / block
    rc = lib.s3r_cmp_attn_topk_fwd(p, p, p, p, p, p, 1, 1, 16, 16, 128, 32, 0.125, None)
    assert rc == -2 and "head_dim" in _lib.last_error()
    rc = lib.s3r_cmp_attn_topk_fwd(p, p, p, p, p, p, 1, 1, 16, 16, 64, 48, 0.125, None)
    assert rc == -2 and "topk" in _lib.last_error()
    rc = lib.s3r_sel_attn_fwd(p, p, p, 1, 0, p, p, None, None, 0, 0, 0, None, None, 1, 1, 64, 64, 64, 48, 8, 0.125, None)
    assert rc == -2 and "block" in _lib.last_error()
    # prologue: NULL output, ragged sequence, head count, LayerNorm parameters only in part, positions without tables
    pro = lambda **kw: lib.s3r_qkv_prologue_fwd(
        kw.get("qkv", p), kw.get("pos"), kw.get("cos"), kw.get("sin"), kw.get("rows", 0), kw.get("qw"), kw.get("qb"),
        kw.get("kw"), kw.get("kb"), 1e-5, p, p, p, p, p, kw.get("v_c", p), 1, kw.get("H", 4), kw.get("N", 32), 64, 16, None)
    assert pro(v_c=None) == -4
    assert pro(N=40) == -1 and "multiple" in _lib.last_error()
    assert pro(H=43) == -2 and "heads" in _lib.last_error()
    assert pro(qw=p) == -4
    assert pro(pos=p) == -4 and "tables" in _lib.last_error()
    # merge arguments must come together
    rc = lib.s3r_sel_attn_fwd(p, p, p, 1, 0, p, p, None, p, 0, 0, 0, None, None, 1, 1, 64, 64, 64, 16, 8, 0.125, None)
    assert rc == -4
    # CSR workspace too small
    need = lib.s3r_csr_workspace_bytes(1, 2, 64, 8, 64)
    assert need > 0
    rc = lib.s3r_build_key_csr(p, p, p, 1, 2, 64, 8, 64, p, need - 1, None)
    assert rc == -6


def test_python_layer_has_no_cpu_fallback():
    import speed3r_b200
    from speed3r_b200 import ops
    q = torch.randn(1, 2, 64, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.flash_attn_topk_func(q, q, q, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.pool_tokens(q, 16, 16)
    m = speed3r_b200.SparseFlashAttentionRope(128, num_heads=2)
    with pytest.raises(RuntimeError):
        m(torch.randn(1, 64, 128))


def test_module_keeps_reference_state_dict_keys_and_init():
    """Keys and gate initialisation of pi3/models/layers/sparse_attention.py:62-86."""
    import speed3r_b200
    m = speed3r_b200.SparseFlashAttentionRope(1024, num_heads=16, qkv_bias=True, qk_norm=True)
    keys = set(m.state_dict().keys())
    assert keys == {"qkv.weight", "qkv.bias", "proj.weight", "proj.bias", "q_norm.weight", "q_norm.bias",
                    "k_norm.weight", "k_norm.bias", "gate.0.weight", "gate.0.bias"}
    assert m.gate[0].weight.abs().max() == 0
    assert torch.equal(m.gate[0].bias.data, torch.tensor([-1.0, 1.0]).repeat(16))
    assert m.block_size == 4 and m.topk == 32


def test_rope_matches_oracle_on_cpu():
    import speed3r_b200
    from oracle import restatement as R
    torch.manual_seed(0)
    x = torch.randn(2, 3, 50, 64)
    pos = torch.randint(0, 37, (2, 50, 2))
    assert torch.equal(speed3r_b200.RoPE2D(100.0)(x, pos), R.rope2d(x, pos, 100.0))
    xb = x.bfloat16()
    assert torch.equal(speed3r_b200.RoPE2D(100.0)(xb, pos), R.rope2d(xb, pos, 100.0))


def test_host_pipeline_chunking():
    """Query chunks of the pinned-host pipeline: whole waves of the compression kernel, full cover, in order."""
    from speed3r_b200.host_pipeline import query_chunks, rows_per_chunk_for
    rows = rows_per_chunk_for(16, 148)
    assert rows == 256 * 37 and (16 * (rows // 256)) % 148 == 0
    assert rows_per_chunk_for(12, 148) == 256 * 37 and rows_per_chunk_for(37, 148) == 256 * 4
    ch = query_chunks(63000, rows)
    assert ch[0] == (0, rows) and ch[-1][1] == 63000 and len(ch) == 7
    assert all(a[1] == b[0] for a, b in zip(ch, ch[1:]))
    assert query_chunks(100, rows) == [(0, 100)]
