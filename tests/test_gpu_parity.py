"""Parity of the CUDA path (called through the C ABI) with the CPU oracle on the same seeded,
bf16-rounded inputs, plus the golden fixtures made from the reference's own kernels."""
import math

import pytest
import torch

from conftest import golden
from _util import assert_bf16_close, assert_idx_match, bf16_round, check_cmp_attn_topk, check_sel_attn
from oracle import restatement as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _status_clean():
    from speed3r_b200 import _lib
    _lib.load()
    _lib.device_status(clear=True)
    yield
    assert _lib.device_status(clear=True) == 0, "a kernel reported a device-side status (timeout / bad index)"


def dev(t, dtype=torch.bfloat16):
    return t.to(DEV, dtype).contiguous()


def randn(seed, *shape):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


# ------------------------------------------------------------------------------------------ pooling
@pytest.mark.parametrize("B,H,T,kernel,stride", [(1, 2, 256, 16, 16), (2, 3, 1041, 32, 16), (1, 16, 2048, 16, 16),
                                                 (1, 1, 100, 16, 16), (1, 2, 333, 32, 32)])
def test_pool_fwd_bwd(B, H, T, kernel, stride):
    from speed3r_b200 import ops
    x, = bf16_round(randn(1, B, H, T, 64))
    ref = R.pool_tokens(x, kernel, stride)
    xg = dev(x).requires_grad_(True)
    out = ops.pool_tokens(xg, kernel, stride)
    assert_bf16_close(out, ref, "pool fwd", max_abs=4e-3, mean_abs=1e-3)
    g, = bf16_round(randn(2, *ref.shape))
    out.backward(dev(g))
    xr = x.clone().requires_grad_(True)
    R.pool_tokens(xr, kernel, stride).backward(g)
    assert_bf16_close(xg.grad, xr.grad, "pool bwd", max_abs=4e-3, mean_abs=1e-3)


def test_pool_packed_qkv_view():
    """Pooling reads the packed projection [B,T,3,H,d] in place through strides."""
    from speed3r_b200 import ops
    B, T, H, d = 2, 320, 4, 64
    qkv, = bf16_round(randn(3, B, T, 3 * H * d))
    ref = R.pool_qkv(qkv, H, 16, 16)
    qg = dev(qkv).view(B, T, 3, H, d)
    for i in range(3):
        out = ops.pool_tokens(qg[:, :, i].permute(0, 2, 1, 3), 16, 16)
        assert_bf16_close(out, ref[i], f"pool packed {i}", max_abs=4e-3, mean_abs=1e-3)


# ------------------------------------------------------------------- compression attention + top-k
def _cmp_case(q, k, v, topk, exact=False, what=""):
    from speed3r_b200 import ops
    q, k, v = bf16_round(q, k, v)
    o_ref, lse_ref, idx_ref = R.cmp_attn_topk(q, k, v, topk)
    S = torch.matmul(q, k.transpose(-1, -2))
    o, lse, idx = ops._cmp_fwd(dev(q), dev(k), dev(v), topk, 1.0 / math.sqrt(q.shape[-1]))
    torch.cuda.synchronize()
    assert_idx_match(idx, idx_ref, S, what + " idx", exact=exact)
    assert_bf16_close(o, o_ref, what + " o_c")
    assert_bf16_close(lse, lse_ref, what + " lse", max_abs=5e-3, mean_abs=1e-3, scale_with_ref=False)


@pytest.mark.parametrize("name", ["cmp_basic", "cmp_ragged", "cmp_rect", "cmp_short", "cmp_ties"])
def test_cmp_attn_topk_golden(name):
    g = golden(name)
    _cmp_case(g["q"], g["k"], g["v"], int(g["topk"]), exact=(name in ("cmp_ties", "cmp_short")), what=name)


@pytest.mark.parametrize("B,H,Nq,Nc,topk", [(1, 4, 1000, 1000, 32), (2, 2, 300, 2500, 16), (1, 2, 257, 129, 32),
                                            (1, 1, 4032, 4032, 32), (1, 2, 5, 40, 8), (1, 2, 700, 900, 1)])
def test_cmp_attn_topk_seeded(B, H, Nq, Nc, topk):
    q, k, v = randn(11, B, H, Nq, 64), randn(12, B, H, Nc, 64), randn(13, B, H, Nc, 64)
    _cmp_case(q, k, v, topk, what=f"seeded {Nq}x{Nc}")


def test_cmp_attn_all_equal_scores():
    """Rows whose logits are all equal (a zero query): the table is columns 0..K-1 in order, and a
    row of equal scores must not slow the scan down (every column ties with the threshold)."""
    from speed3r_b200 import ops
    B, H, Nq, Nc, K = 1, 2, 300, 2000, 32
    q = torch.zeros(B, H, Nq, 64)
    q[:, :, ::2] = randn(81, B, H, (Nq + 1) // 2, 64)          # odd rows stay zero
    k, v = randn(82, B, H, Nc, 64), randn(83, B, H, Nc, 64)
    _cmp_case(q, k, v, K, what="equal-scores")
    _, _, idx = ops._cmp_fwd(dev(q), dev(k), dev(v), K, 0.125)
    assert torch.equal(idx[:, :, 1::2].cpu(), torch.arange(K, dtype=torch.int32).expand(B, H, Nq // 2, K))


def test_cmp_attn_large_logits_and_rescale():
    """Row maxima that grow along the key axis force the lazy O rescale path."""
    B, H, N = 1, 2, 1024
    q, k, v = randn(21, B, H, N, 64), randn(22, B, H, N, 64), randn(23, B, H, N, 64)
    k = k * torch.linspace(0.2, 3.0, N).view(1, 1, N, 1)
    _cmp_case(q * 1.5, k, v, 32, what="rescale")


def test_cmp_attn_matches_device_check_at_scale():
    """100 views x 1008 tokens (Nc = 6300), all 16 heads: tensor-core kernel vs the SIMT restatement."""
    from speed3r_b200 import ops
    B, H, N = 1, 16, 6300
    g = torch.Generator(device=DEV).manual_seed(5)
    q, k, v = (torch.nn.functional.layer_norm(torch.randn(B, H, N, 64, device=DEV, generator=g), (64,)).bfloat16()
               for _ in range(3))
    o, lse, idx = ops._cmp_fwd(q, k, v, 32, 0.125)
    o2, lse2, idx2 = check_cmp_attn_topk(q, k, v, 32, 0.125)
    torch.cuda.synchronize()
    assert_bf16_close(o, o2, "o_c vs device check")
    assert_bf16_close(lse, lse2, "lse vs device check", max_abs=5e-3, mean_abs=1e-3, scale_with_ref=False)
    frac = (idx != idx2).float().mean().item()
    assert frac < 2e-3, f"{frac:.2e} of index entries differ from the device check"
    for h in (0, 7, 15):            # tie check of the differing entries on a few heads
        S = torch.matmul(q[0, h].float(), k[0, h].float().t()).cpu()
        assert_idx_match(idx[0, h], idx2[0, h], S, f"scale idx head {h}")


# ---------------------------------------------------------------------------- selection attention
def _rand_idx(seed, B, H, nqb, nkb, K):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.stack([torch.stack([
        (torch.randperm(nkb, generator=g)[:K] if nkb >= K else torch.randint(0, nkb, (K,), generator=g))
        for _ in range(nqb)]) for _ in range(H)]) for _ in range(B)]).int()


@pytest.mark.parametrize("name", ["sel_basic", "sel_k32", "sel_dup", "sel_neg", "sel_bs64"])
def test_sel_attn_golden(name):
    from speed3r_b200 import ops
    g = golden(name)
    q, k, v = bf16_round(g["q"], g["k"], g["v"])
    o_ref, lse_ref = R.sel_attn(q, k, v, g["idx"], int(g["block"]))
    o = ops.topk_blocksparse_attention(dev(q), dev(k), dev(v), g["idx"].to(DEV), int(g["block"]))
    assert_bf16_close(o, o_ref, name + " o_s")
    # the fixture itself (fp32 inputs) is within bf16 input-rounding distance as well
    assert_bf16_close(o, g["o"], name + " o_s vs fixture", max_abs=6e-2, mean_abs=6e-3)


@pytest.mark.parametrize("B,H,T,Bs,K", [(1, 2, 1008, 16, 32), (2, 2, 1041, 16, 32), (1, 3, 1041, 64, 16),
                                        (1, 2, 800, 32, 8), (1, 1, 48, 16, 32), (1, 2, 2048, 16, 33)])
def test_sel_attn_seeded_fwd_bwd(B, H, T, Bs, K):
    from speed3r_b200 import ops
    q, k, v = bf16_round(randn(31, B, H, T, 64), randn(32, B, H, T, 64), randn(33, B, H, T, 64))
    nb = (T + Bs - 1) // Bs
    idx = _rand_idx(34, B, H, nb, nb, K)
    idx[:, :, 0, 0] = nb - 1                   # the partial last block, when T % Bs != 0
    idx[:, :, -1, 1] = nb - 1
    if K >= 4:
        idx[:, :, 1, 2] = -1                   # skipped
        idx[:, :, 1, 3] = nb + 5               # out of range: skipped
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_ref, lse_ref = R.sel_attn(qr, kr, vr, idx, Bs)
    qg, kg, vg = (dev(t).requires_grad_(True) for t in (q, k, v))
    o = ops.topk_blocksparse_attention(qg, kg, vg, idx.to(DEV), Bs)
    assert_bf16_close(o, o_ref, "o_s")
    o_chk, lse_chk = check_sel_attn(qg.detach(), kg.detach(), vg.detach(), idx.to(DEV), Bs)
    assert_bf16_close(o_chk, o_ref, "device check o_s")
    assert_bf16_close(lse_chk, lse_ref, "device check lse", max_abs=5e-3, mean_abs=1e-3, scale_with_ref=False)
    do, = bf16_round(randn(35, B, H, T, 64))
    o_ref.backward(do)
    o.backward(dev(do))
    assert_bf16_close(qg.grad, qr.grad, "dq")
    assert_bf16_close(kg.grad, kr.grad, "dk")
    assert_bf16_close(vg.grad, vr.grad, "dv")


def test_sel_attn_backward_sink_blocks():
    """Key blocks that every query block selects (long CSR segments: the register-chunked list walk of the
    dK/dV kernel crosses many 32-entry chunks) next to blocks nobody selects (empty segments)."""
    from speed3r_b200 import ops
    B, H, T, Bs, K = 1, 2, 3200, 16, 8
    q, k, v = bf16_round(randn(41, B, H, T, 64), randn(42, B, H, T, 64), randn(43, B, H, T, 64))
    nb = T // Bs                                  # 200 query blocks
    idx = _rand_idx(44, B, H, nb, nb // 2, K)     # the upper half of the key blocks is never selected ...
    idx[:, :, :, 0] = 0                           # ... block 0 by every query block
    idx[:, :, :, 1] = 7                           # and block 7 as well
    idx[:, :, ::3, 2] = nb - 1                    # every third one the last block
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_ref, _ = R.sel_attn(qr, kr, vr, idx, Bs)
    qg, kg, vg = (dev(t).requires_grad_(True) for t in (q, k, v))
    o = ops.topk_blocksparse_attention(qg, kg, vg, idx.to(DEV), Bs)
    assert_bf16_close(o, o_ref, "o_s")
    do, = bf16_round(randn(45, B, H, T, 64))
    o_ref.backward(do)
    o.backward(dev(do))
    assert_bf16_close(qg.grad, qr.grad, "dq")
    assert_bf16_close(kg.grad, kr.grad, "dk")
    assert_bf16_close(vg.grad, vr.grad, "dv")
    assert float(kg.grad[:, :, (nb // 2 + 1) * Bs:(nb - 1) * Bs].abs().max()) == 0.0   # unselected blocks: exact zeros


@pytest.mark.parametrize("B,H,T,Lc,Sc,Bs,K", [(1, 2, 4096, 32, 16, 64, 16), (2, 2, 2112, 32, 16, 64, 16),
                                              (1, 2, 3072, 16, 16, 64, 8), (1, 1, 1024, 64, 16, 64, 32)])
def test_extension_setting_block_ranking(B, H, T, Lc, Sc, Bs, K):
    """Compressed keys finer than selection blocks (windows of Lc every Sc tokens, blocks of Bs = 4*Sc): the
    table ranks blocks by the softmax mass of their own compressed keys.  The oracle is the definition
    (`block_rank_scores`); entries may differ only where the competing block scores are closer than 1e-3."""
    from speed3r_b200 import ops
    q, k, v = bf16_round(randn(51, B, H, T, 64), randn(52, B, H, T, 64), randn(53, B, H, T, 64))
    gate, = bf16_round(torch.sigmoid(randn(54, B, H, T, 2)))
    group, take = Bs // Sc, (Bs - Lc) // Sc + 1
    q_c, k_c, v_c = R.pool_tokens(q, Bs, Bs), R.pool_tokens(k, Lc, Sc), R.pool_tokens(v, Lc, Sc)
    q_c, k_c, v_c = bf16_round(q_c, k_c, v_c)
    o_ref, lse_ref, idx_ref = R.cmp_attn_topk(q_c, k_c, v_c, K, rank_group=(group, take))
    o, idx = ops.flash_attn_blocktopk_func(dev(q_c), dev(k_c), dev(v_c), K, group, take)
    assert_bf16_close(o, o_ref, "o_c")
    idx = idx.cpu()
    Nb = (k_c.shape[2] - take) // group + 1
    assert int(idx.max()) < Nb and int(idx.min()) >= 0
    scores = R.block_rank_scores(torch.matmul(q_c.float(), k_c.float().transpose(-1, -2)), 0.125, group, take)
    kk = min(K, Nb)
    mism = idx[..., :kk] != idx_ref[..., :kk]
    if mism.any():                                   # only near-ties may differ
        a = torch.gather(scores, -1, idx[..., :kk].long())
        b = torch.gather(scores, -1, idx_ref[..., :kk].long())
        assert float((a - b).abs()[mism].max()) < 1e-3, "block table differs beyond near-ties"
        assert mism.float().mean() < 0.02
    if Nb < K:
        assert torch.all(idx[..., Nb:] == Nb - 1)    # padding, as the column table pads with Nc-1
    # the whole op at this setting, forward and backward, given the table the GPU selected
    qg, kg, vg = (dev(t).requires_grad_(True) for t in (q, k, v))
    y, idx_op = ops.sparse_attention_op(qg, kg, vg, dev(gate), Bs, K, Lc, Sc)
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    qc_r, kc_r, vc_r = R.pool_tokens(qr, Bs, Bs), R.pool_tokens(kr, Lc, Sc), R.pool_tokens(vr, Lc, Sc)
    oc_r, _, _ = R.cmp_attn_topk(qc_r, kc_r, vc_r, K, rank_group=(group, take))
    os_r, _ = R.sel_attn(qr, kr, vr, idx_op.cpu(), Bs)
    y_ref = R.gated_merge(gate, oc_r, os_r, Bs)
    assert_bf16_close(y, y_ref, "y")
    dy, = bf16_round(randn(55, B, T, H * 64))
    y_ref.backward(dy)
    y.backward(dev(dy))
    assert_bf16_close(qg.grad, qr.grad, "dq")
    assert_bf16_close(kg.grad, kr.grad, "dk")
    assert_bf16_close(vg.grad, vr.grad, "dv")


def test_sel_attn_merge_fused_fwd_bwd():
    from speed3r_b200 import ops
    B, H, T, Bs, K = 2, 4, 656, 16, 32
    q, k, v = bf16_round(randn(41, B, H, T, 64), randn(42, B, H, T, 64), randn(43, B, H, T, 64))
    nb = T // Bs
    idx = _rand_idx(44, B, H, nb, nb, K)
    gate_flat, = bf16_round(torch.sigmoid(randn(45, B, T, 2 * H)))
    o_c, = bf16_round(randn(46, B, H, nb, 64))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, gate_flat, o_c)]
    qr, kr, vr, gr, ocr = leaves
    o_s_ref, _ = R.sel_attn(qr, kr, vr, idx, Bs)
    y_ref = R.gated_merge(gr.view(B, T, H, 2).permute(0, 2, 1, 3), ocr, o_s_ref, Bs)
    gl = [dev(t).requires_grad_(True) for t in (q, k, v, gate_flat, o_c)]
    qg, kg, vg, gg, ocg = gl
    y = ops.sel_attn_merge(qg, kg, vg, idx.to(DEV), gg.view(B, T, H, 2).permute(0, 2, 1, 3), ocg, Bs)
    assert_bf16_close(y, y_ref, "merged y")
    dy, = bf16_round(randn(47, B, T, H * 64))
    y_ref.backward(dy)
    y.backward(dev(dy))
    for name, a, b in zip(("dq", "dk", "dv", "dgate", "do_c"), gl, leaves):
        assert_bf16_close(a.grad, b.grad, name)


def test_sel_attn_chunked_kv_matches_dense():
    """K/V stored as sequence chunks (the layout an all-gather leaves) give identical results."""
    from speed3r_b200 import ops
    B, H, T, Bs, K, G = 1, 2, 1024, 16, 32, 4
    g = torch.Generator(device=DEV).manual_seed(7)
    q, k, v = (torch.randn(B, H, T, 64, device=DEV, generator=g).bfloat16() for _ in range(3))
    idx = _rand_idx(51, B, H, T // Bs, T // Bs, K).to(DEV)
    o_d, lse_d, _ = ops._sel_fwd(q, k, v, idx, None, None, Bs, 0.125, True, True, 1)
    kc = k.view(B, H, G, T // G, 64).permute(2, 0, 1, 3, 4).contiguous()
    vc = v.view(B, H, G, T // G, 64).permute(2, 0, 1, 3, 4).contiguous()
    o_c, lse_c, _ = ops._sel_fwd(q, kc, vc, idx, None, None, Bs, 0.125, True, True, G)
    assert torch.equal(o_d, o_c) and torch.equal(lse_d, lse_c)


def test_host_pipeline_matches_device_call():
    """Pinned-host entry: K/V by head group, queries in chunks (one of them ragged), three streams.
    Every query row sees the same keys in the same order, so the result is bit-identical to the one-shot
    device call, twice in a row (the second call reuses the device buffers)."""
    from speed3r_b200 import ops, HostPipeline
    H, Bs, K = 4, 16, 32
    T = Bs * (2 * 256 + 100)
    g = torch.Generator().manual_seed(11)
    ln = lambda t: torch.nn.functional.layer_norm(t, (64,))
    hq, hk, hv = (ln(torch.randn(1, H, T, 64, generator=g)).bfloat16().pin_memory() for _ in range(3))
    hgate = torch.sigmoid(torch.randn(1, H, T, 2, generator=g)).bfloat16().pin_memory()
    q, k, v, gate = (t.to(DEV) for t in (hq, hk, hv, hgate))
    qc, kc, vc = (ops.pool_tokens(t, Bs, Bs) for t in (q, k, v))
    o_c, idx = ops.flash_attn_topk_func(qc, kc, vc, K)
    y_ref = ops.sel_attn_merge(q, k, v, idx, gate, o_c, Bs).cpu()
    pipe = HostPipeline(H, T, 64, Bs, K, device=DEV, rows_per_chunk=256, heads_per_copy=3)
    assert len(pipe.chunks()) == 3
    for _ in range(2):
        hy = torch.zeros(1, T, H * 64, dtype=torch.bfloat16).pin_memory()
        pipe(hq, hk, hv, hgate, hy)
        torch.cuda.synchronize()
        assert torch.equal(hy, y_ref)
    with pytest.raises(RuntimeError):
        pipe(hq.clone(), hk, hv, hgate, hy)      # not pinned


def test_sel_attn_deterministic():
    from speed3r_b200 import ops
    B, H, T, Bs, K = 1, 4, 2048, 16, 32
    g = torch.Generator(device=DEV).manual_seed(9)
    q, k, v, do = (torch.randn(B, H, T, 64, device=DEV, generator=g).bfloat16() for _ in range(4))
    idx = _rand_idx(52, B, H, T // Bs, T // Bs, K).to(DEV)
    outs = []
    for _ in range(2):
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = ops.topk_blocksparse_attention(qg, kg, vg, idx, Bs)
        o.backward(do)
        outs.append((o.detach(), qg.grad, kg.grad, vg.grad))
    for a, b in zip(*outs):
        assert torch.equal(a, b), "two runs on identical inputs differ"


# ----------------------------------------------------------------------------------- CSR, backward
@pytest.mark.parametrize("B,H,Nq,K,Nkb", [(1, 2, 64, 8, 64), (2, 3, 100, 32, 100), (1, 1, 16, 32, 16)])
def test_key_csr_matches_oracle(B, H, Nq, K, Nkb):
    from speed3r_b200 import ops
    idx = _rand_idx(61, B, H, Nq, Nkb, K)
    idx[:, :, 0, 0] = -1
    idx[:, :, 1, 1] = Nkb + 3
    if Nkb < K:
        idx[..., K // 2:] = Nkb - 1
    offs_ref, qids_ref = R.key_centric_csr(idx, Nkb)
    offs, qids = ops.build_key_csr(idx.to(DEV), Nkb)
    assert torch.equal(offs.cpu(), offs_ref)
    n = qids_ref.shape[-1]
    for b in range(B):
        for h in range(H):
            tot = int(offs_ref[b, h, -1])
            assert torch.equal(qids[b, h, :tot].cpu(), qids_ref[b, h, :tot])


def test_key_csr_sink_blocks():
    """Key blocks that (nearly) every query block selects - attention sinks - give segments of thousands
    of entries: the build must order them as the oracle does (all three length classes of its sort:
    a warp, a CTA in shared memory, the ordered walk over the table) and do so in milliseconds."""
    import time
    from speed3r_b200 import ops
    B, H, Nq, K, Nkb = 1, 2, 6000, 32, 6000
    idx = _rand_idx(62, B, H, Nq, Nkb, K - 2)
    sink = torch.zeros(B, H, Nq, 1, dtype=torch.int32)                         # block 0: listed by everyone (6000)
    g = torch.Generator().manual_seed(63)
    mid = torch.where(torch.rand(B, H, Nq, 1, generator=g) < 0.3, 7, -1).int()  # block 7: ~1800 entries (+ random)
    idx = torch.cat((idx[..., :5], sink, idx[..., 5:], mid), -1).contiguous()
    offs_ref, qids_ref = R.key_centric_csr(idx, Nkb)
    assert int(offs_ref[0, 0, 1] - offs_ref[0, 0, 0]) >= Nq and 1000 < int(offs_ref[0, 0, 8] - offs_ref[0, 0, 7]) < 4096
    idx_d = idx.to(DEV)
    ops.build_key_csr(idx_d, Nkb)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    offs, qids = ops.build_key_csr(idx_d, Nkb)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert torch.equal(offs.cpu(), offs_ref)
    for h in range(H):
        tot = int(offs_ref[0, h, -1])
        assert torch.equal(qids[0, h, :tot].cpu(), qids_ref[0, h, :tot])
    assert dt < 0.05, f"index build with sink blocks took {dt * 1e3:.1f} ms"


@pytest.mark.parametrize("name", ["cmp_basic", "cmp_ragged"])
def test_cmp_attn_backward_golden(name):
    from speed3r_b200 import ops
    g = golden(name)
    q, k, v, do = bf16_round(g["q"], g["k"], g["v"], g["do"])
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_ref, _, _ = R.cmp_attn_topk(qr, kr, vr, int(g["topk"]))
    o_ref.backward(do)
    qg, kg, vg = (dev(t).requires_grad_(True) for t in (q, k, v))
    o, idx = ops.flash_attn_topk_func(qg, kg, vg, int(g["topk"]))
    o.backward(dev(do))
    assert_bf16_close(qg.grad, qr.grad, "dq_c")
    assert_bf16_close(kg.grad, kr.grad, "dk_c")
    assert_bf16_close(vg.grad, vr.grad, "dv_c")


@pytest.mark.parametrize("B,H,Nq,Nc", [(2, 2, 203, 391), (1, 2, 1100, 777), (1, 1, 40, 50), (1, 1, 64, 17)])
def test_cmp_attn_backward_seeded_rect(B, H, Nq, Nc):
    from speed3r_b200 import ops
    q, k, v, do = bf16_round(randn(71, B, H, Nq, 64), randn(72, B, H, Nc, 64), randn(73, B, H, Nc, 64),
                             randn(74, B, H, Nq, 64))
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    R.cmp_attn_topk(qr, kr, vr, 16)[0].backward(do)
    qg, kg, vg = (dev(t).requires_grad_(True) for t in (q, k, v))
    ops.flash_attn_topk_func(qg, kg, vg, 16)[0].backward(dev(do))
    assert_bf16_close(qg.grad, qr.grad, "dq_c")
    assert_bf16_close(kg.grad, kr.grad, "dk_c")
    assert_bf16_close(vg.grad, vr.grad, "dv_c")


@pytest.mark.parametrize("name", ["sel_basic", "sel_k32", "sel_dup", "sel_bs64"])
def test_sel_attn_backward_golden(name):
    from speed3r_b200 import ops
    g = golden(name)
    q, k, v, do = bf16_round(g["q"], g["k"], g["v"], g["do"])
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    R.sel_attn(qr, kr, vr, g["idx"], int(g["block"]))[0].backward(do)
    qg, kg, vg = (dev(t).requires_grad_(True) for t in (q, k, v))
    ops.topk_blocksparse_attention(qg, kg, vg, g["idx"].to(DEV), int(g["block"])).backward(dev(do))
    assert_bf16_close(qg.grad, qr.grad, name + " dq")
    assert_bf16_close(kg.grad, kr.grad, name + " dk")
    assert_bf16_close(vg.grad, vr.grad, name + " dv")


# ------------------------------------------------------------------------ whole op / whole module
def test_cfg1_op_forward():
    """BASELINE config 1: B=1, T=2048 (8 views x 256), 16 heads, d=64, seed 0, 16/16/16/32."""
    from speed3r_b200 import ops
    torch.manual_seed(0)
    B, H, T, d, Bs, K = 1, 16, 2048, 64, 16, 32
    q, k, v = torch.randn(B, H, T, d), torch.randn(B, H, T, d), torch.randn(B, H, T, d)
    gate = torch.sigmoid(torch.randn(B, H, T, 2))
    q, k, v, gate = bf16_round(q, k, v, gate)
    # oracle on the bf16-rounded inputs, with pooled tensors rounded to bf16 as the kernels see them
    q_c, k_c, v_c = bf16_round(*(R.pool_tokens(t, Bs, Bs) for t in (q, k, v)))
    qg, kg, vg, gg = dev(q), dev(k), dev(v), dev(gate)
    qc, kc, vc = (ops.pool_tokens(t, Bs, Bs) for t in (qg, kg, vg))
    for a, b in zip((qc, kc, vc), (q_c, k_c, v_c)):
        assert_bf16_close(a, b, "cfg1 pooled", max_abs=4e-3, mean_abs=5e-4)
    # from here on the oracle sees exactly the pooled tensors the kernels see
    q_c, k_c, v_c = (t.cpu().float() for t in (qc, kc, vc))
    o_c_ref, _, idx_ref = R.cmp_attn_topk(q_c, k_c, v_c, K)
    o_c, idx = ops.flash_attn_topk_func(qc, kc, vc, K)
    assert_idx_match(idx, idx_ref, torch.matmul(q_c, k_c.transpose(-1, -2)), "cfg1 idx")
    assert_bf16_close(o_c, o_c_ref, "cfg1 o_c")
    y = ops.sel_attn_merge(qg, kg, vg, idx, gg, o_c, Bs)
    o_s_ref, _ = R.sel_attn(q, k, v, idx.cpu(), Bs)
    y_ref = R.gated_merge(gate, o_c_ref, o_s_ref, Bs)
    assert_bf16_close(y, y_ref, "cfg1 y")


def _module_pair(g, backward=False):
    import speed3r_b200
    heads = int(g["heads"])
    dim = g["x"].shape[-1]
    m = speed3r_b200.SparseFlashAttentionRope(dim, num_heads=heads, qkv_bias=True, proj_bias=True, qk_norm=True,
                                              rope=speed3r_b200.RoPE2D(100.0))
    sd = {k[len("param."):]: v for k, v in g.items() if k.startswith("param.")}
    m.load_state_dict(sd, strict=True)
    return m.to(DEV), sd, heads


def test_module_forward_golden():
    """Whole module in bf16 autocast against the fp32 oracle (itself pinned to the reference's
    output for this fixture).  bf16 noise can flip near-tie selections, so the oracle is given the
    table the GPU selected; the agreement of that table with the fp32 selection is checked apart."""
    g = golden("module_fwd")
    m, sd, heads = _module_pair(g)
    m.record_idx = True
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(g["x"].to(DEV), xpos=g["xpos"].to(DEV))
    idx = m.last_idx.cpu()
    y_ref, aux = R.module_forward(sd, g["x"], g["xpos"], heads, return_aux=True, idx_override=idx)
    # three bf16 GEMMs, LayerNorm and RoPE in bf16 against fp32: looser than the op-level bound
    assert_bf16_close(y, y_ref, "module y", max_abs=6e-2, mean_abs=8e-3)
    _, aux0 = R.module_forward(sd, g["x"], g["xpos"], heads, return_aux=True)
    same = (torch.sort(idx, -1).values == torch.sort(aux0["idx"], -1).values).float().mean().item()
    assert same > 0.85, f"only {same:.2%} of the selected blocks agree with the fp32 selection"


@pytest.mark.parametrize("with_norm,with_pos,H,Bs", [(True, True, 16, 16), (False, True, 2, 16), (True, False, 5, 4)])
def test_qkv_prologue_matches_separate_steps(with_norm, with_pos, H, Bs):
    """The one-pass prologue against the module's separate PyTorch steps (LayerNorm under autocast, RoPE2D in
    bf16, the pooling kernel): v and its block means bit-equal; q, k and their pooled forms equal up to the
    last bf16 bit of the LayerNorm (different fp32 summation order)."""
    import speed3r_b200
    from speed3r_b200 import ops
    B, N, d = 2, 16 * 24, 64
    g = torch.Generator(device=DEV).manual_seed(5)
    qkv = (torch.randn(B, N, 3 * H * d, device=DEV, generator=g) * 1.5 + 0.3).bfloat16()
    pos = torch.randint(0, 37, (B, N, 2), device=DEV, generator=g) if with_pos else None
    rope = speed3r_b200.RoPE2D(100.0)
    qn = torch.nn.LayerNorm(d).to(DEV) if with_norm else torch.nn.Identity()
    kn = torch.nn.LayerNorm(d).to(DEV) if with_norm else torch.nn.Identity()
    if with_norm:
        with torch.no_grad():
            for m in (qn, kn):
                m.weight.copy_(1 + 0.2 * torch.randn(d, device=DEV, generator=g))
                m.bias.copy_(0.1 * torch.randn(d, device=DEV, generator=g))
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        q_t, k_t, v_t = (qkv.view(B, N, 3, H, d)[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        q_c, k_c, v_c = (ops.pool_tokens(t, Bs, Bs) for t in (q_t, k_t, v_t))
        q_c, k_c = qn(q_c).to(qkv.dtype), kn(k_c).to(qkv.dtype)
        q, k = qn(q_t).to(qkv.dtype), kn(k_t).to(qkv.dtype)
        if with_pos:
            pos_c = pos.view(B, N // Bs, Bs, 2).float().mean(dim=2).int()
            q_c, k_c, q, k = rope(q_c, pos_c), rope(k_c, pos_c), rope(q, pos), rope(k, pos)
        cos = sin = None
        if with_pos:
            cos, sin = rope._cos_sin(d // 2, rope._seq_len(pos), qkv.device, qkv.dtype)
        norms = ((qn.weight, qn.bias, qn.eps), (kn.weight, kn.bias, kn.eps)) if with_norm else (None, None)
        fq, fk, fv, fqc, fkc, fvc = ops.qkv_prologue(qkv, H, Bs, pos, cos, sin, norms[0], norms[1])
    assert torch.equal(fv, v_t.contiguous()) and torch.equal(fvc, v_c)
    for name, a, b in (("q", fq, q), ("k", fk, k), ("q_c", fqc, q_c), ("k_c", fkc, k_c)):
        assert a.shape == b.shape, name
        same = (a == b).float().mean().item()
        assert same > (0.98 if with_norm else 0.9999), f"{name}: only {same:.4%} of the elements are bit-equal"
        assert_bf16_close(a, b.float(), name, max_abs=4e-2, mean_abs=1e-3)


def test_qkv_prologue_against_oracle():
    """The prologue kernel against the fp32 CPU restatement on the module fixture's projection (bf16-rounded):
    bf16 rounding of LayerNorm and of the three rotary roundings is the only difference."""
    import speed3r_b200
    from speed3r_b200 import ops
    g = golden("module_fwd")
    sd = {k[len("param."):]: v for k, v in g.items() if k.startswith("param.")}
    heads = int(g["heads"])
    qkv, = bf16_round(torch.nn.functional.linear(g["x"], sd["qkv.weight"], sd["qkv.bias"]))
    ref = R.qkv_prologue(qkv, heads, 16, g["xpos"], (sd["q_norm.weight"], sd["q_norm.bias"]),
                         (sd["k_norm.weight"], sd["k_norm.bias"]))
    rope = speed3r_b200.RoPE2D(100.0)
    xpos = g["xpos"].to(DEV)
    cos, sin = rope._cos_sin(32, rope._seq_len(xpos), torch.device(DEV), torch.bfloat16)
    out = ops.qkv_prologue(dev(qkv), heads, 16, xpos, cos, sin,
                           (sd["q_norm.weight"], sd["q_norm.bias"], 1e-5), (sd["k_norm.weight"], sd["k_norm.bias"], 1e-5))
    for name, a, b in zip(("q", "k", "v", "q_c", "k_c", "v_c"), out, ref):
        # the rotary angles are rounded to bf16 before cos/sin on both sides; values reach ~4
        assert_bf16_close(a, b, "prologue " + name, max_abs=6e-2, mean_abs=6e-3)


def test_module_forward_without_grad_uses_fused_prologue_and_matches():
    """Under no_grad the module runs the one-pass prologue; its output equals the grad-enabled path's up to
    bf16 rounding, and agrees with the oracle as the other path does."""
    g = golden("module_fwd")
    m, sd, heads = _module_pair(g)
    m.record_idx = True
    x, xpos = g["x"].to(DEV), g["xpos"].to(DEV)
    assert m._can_fuse_prologue(torch.empty(0), x, xpos, x.shape[1], m.block_size ** 2, x.shape[-1] // heads) is False
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y_sep = m(x, xpos=xpos)
        idx_sep = m.last_idx.cpu()
        with torch.no_grad():
            assert m._can_fuse_prologue(torch.empty(0), x, xpos, x.shape[1], m.block_size ** 2, x.shape[-1] // heads)
            y = m(x, xpos=xpos)
    idx = m.last_idx.cpu()
    y_ref, _ = R.module_forward(sd, g["x"], g["xpos"], heads, return_aux=True, idx_override=idx)
    assert_bf16_close(y, y_ref, "module y (fused prologue)", max_abs=6e-2, mean_abs=8e-3)
    same = (torch.sort(idx, -1).values == torch.sort(idx_sep, -1).values).float().mean().item()
    assert same > 0.97, f"only {same:.2%} of the selected blocks agree between the two prologues"
    assert_bf16_close(y, y_sep.detach().float(), "fused vs separate", max_abs=6e-2, mean_abs=4e-3)


def test_module_backward_golden():
    g = golden("module_bwd")
    m, sd, heads = _module_pair(g)
    m.record_idx = True
    x = g["x"].to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x, xpos=g["xpos"].to(DEV))
    y.float().backward(g["dy"].to(DEV))
    p = {k: v.clone().requires_grad_(True) for k, v in sd.items()}
    xr = g["x"].clone().requires_grad_(True)
    y_ref = R.module_forward(p, xr, g["xpos"], heads, idx_override=m.last_idx.cpu())
    y_ref.backward(g["dy"])
    assert_bf16_close(y, y_ref, "module y", max_abs=6e-2, mean_abs=8e-3)
    assert_bf16_close(x.grad, xr.grad, "module dx", max_abs=6e-2, mean_abs=8e-3)
    for k, prm in m.named_parameters():
        assert_bf16_close(prm.grad, p[k].grad, "grad " + k, max_abs=6e-2, mean_abs=1e-2)


def test_module_under_checkpoint_recompute_is_deterministic():
    """Pi3_Sparse wraps the block in activation checkpointing when training (pi3_sparse.py:252-253):
    the recomputed forward must select the same blocks."""
    import speed3r_b200
    from torch.utils.checkpoint import checkpoint
    torch.manual_seed(3)
    m = speed3r_b200.SparseFlashAttentionRope(256, num_heads=4, qkv_bias=True, qk_norm=True,
                                              rope=speed3r_b200.RoPE2D()).to(DEV)
    x = torch.randn(1, 1024, 256, device=DEV, requires_grad=True)
    ys, xs = torch.meshgrid(torch.arange(32), torch.arange(32), indexing="ij")
    xpos = torch.stack([ys, xs], -1).view(1, -1, 2).to(DEV)
    grads = []
    for use_ckpt in (False, True):
        x.grad = None
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = checkpoint(m, x, None, xpos, use_reentrant=False) if use_ckpt else m(x, xpos=xpos)
        y.float().square().mean().backward()
        grads.append(x.grad.clone())
    assert torch.equal(grads[0], grads[1])


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier nobody arrives on must end by itself after its limit (1 ms here), return
    normally and raise the wait-timeout bit of the status word (probe in the tests-only library)."""
    import ctypes as C
    from speed3r_b200 import _lib
    chk = _lib.load_check()
    word = C.c_uint32(0)
    assert chk.s3r_device_status(C.byref(word), 1) == 0
    waited = torch.zeros(1, device=DEV, dtype=torch.int64)
    rc = chk.s3r_check_wait_gives_up(1_000_000, waited.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert chk.s3r_device_status(C.byref(word), 1) == 0
    assert word.value & 1, "the wait ended without raising S3R_STATUS_WAIT_TIMEOUT"
    assert 1_000_000 <= waited.item() < 50_000_000, f"waited {waited.item()} ns for a 1 ms limit"
    assert chk.s3r_device_status(C.byref(word), 1) == 0 and word.value == 0


def test_prologue_flags_positions_outside_its_tables():
    """A position beyond the cos/sin tables is clamped (no fault) and raises the bad-index status bit."""
    import speed3r_b200
    from speed3r_b200 import _lib, ops
    B, N, H, d, Bs = 1, 64, 2, 64, 16
    qkv = dev(randn(95, B, N, 3 * H * d))
    pos = torch.randint(0, 8, (B, N, 2), generator=torch.Generator().manual_seed(96)).to(DEV)
    cos, sin = speed3r_b200.RoPE2D(100.0)._cos_sin(d // 2, 8, torch.device(DEV), torch.bfloat16)
    _lib.device_status(clear=True)
    ops.qkv_prologue(qkv, H, Bs, pos, cos, sin)
    assert _lib.device_status(clear=True) == 0
    pos[0, 5, 1] = 11                                  # outside the 8-row tables
    ops.qkv_prologue(qkv, H, Bs, pos, cos, sin)
    assert _lib.device_status(clear=True) == 2


def test_rejects_cpu_and_fp32():
    from speed3r_b200 import ops
    q = torch.randn(1, 1, 32, 64)
    with pytest.raises(RuntimeError):
        ops.flash_attn_topk_func(q.bfloat16(), q.bfloat16(), q.bfloat16(), 8)       # CPU tensors
    with pytest.raises(RuntimeError):
        ops.flash_attn_topk_func(q.to(DEV), q.to(DEV), q.to(DEV), 8)                # fp32
