"""Generate the golden fixtures in this folder by running the REFERENCE's own code on CPU.

The reference's kernels are Triton; with ``TRITON_INTERPRET=1`` they execute on CPU
tensors (fp32 only: bf16 is not handled correctly by the interpreter).  This script
imports the reference package from the path given by ``--reference`` (it is not
vendored and is never needed at test time), runs seeded inputs through

* ``forward_with_topk`` / ``_flash_attn_backward``      (flash_attention_topk.py:156,515)
* ``_topk_blocksparse_attention_fwd`` / ``_bwd``        (topk_blocksparse_attention.py:852,907)
* ``SparseFlashAttentionRope.forward``                  (sparse_attention.py:90-141)

and stores inputs and outputs as compressed ``.npz`` files.  The module-level cases
swap the public ``topk_blocksparse_attention`` wrapper (which asserts bf16,
topk_blocksparse_attention.py:1053) for a call to the un-asserted inner functions; the
arithmetic is untouched.

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/speed3r [--only NAME]
"""
from __future__ import annotations

import argparse
import math
import os
import sys
import time

os.environ.setdefault("TRITON_INTERPRET", "1")
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _ref(reference):
    sys.dont_write_bytecode = True
    sys.path.insert(0, reference)
    import pi3.models.sparse_attn.flash_attention_topk as fat
    import pi3.models.sparse_attn.topk_blocksparse_attention as tba
    import pi3.models.layers.sparse_attention as sa
    from pi3.models.layers.pos_embed import RoPE2D
    return fat, tba, sa, RoPE2D


def save(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = v
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({os.path.getsize(path) / 1024:.0f} KiB)", flush=True)


def gen_inputs(seed, *shape):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g)


# ---------------------------------------------------------------- compression attention + top-k
def case_cmp(fat, name, seed, B, H, Nq, Nc, K, tie_mode=False, backward=False):
    d = 64
    if tie_mode:
        # small-integer entries: many exactly equal logits -> exercises (value desc, column asc)
        g = torch.Generator().manual_seed(seed)
        q = torch.randint(-1, 2, (B, H, Nq, d), generator=g).float()
        k = torch.randint(-1, 2, (B, H, Nc, d), generator=g).float()
        k[:, :, 5] = k[:, :, 3]          # duplicate key rows: exact ties for every query
        k[:, :, Nc - 1] = k[:, :, 3]
        v = torch.randn(B, H, Nc, d, generator=g)
    else:
        q, k, v = gen_inputs(seed, B, H, Nq, d), gen_inputs(seed + 1, B, H, Nc, d), gen_inputs(seed + 2, B, H, Nc, d)
    o, lse, idx, scale = fat.forward_with_topk(q, k, v, K)
    out = dict(q=q, k=k, v=v, o=o, lse=lse[:, :, :Nq], idx=idx, topk=np.int32(K))
    if backward:
        do = gen_inputs(seed + 3, B, H, Nq, d)
        dq, dk, dv = fat._flash_attn_backward(o, do, lse, q, k, v, scale)
        out.update(do=do, dq=dq, dk=dk, dv=dv)
    save(name, **out)


# ---------------------------------------------------------------- selection attention
def case_sel(tba, name, seed, B, H, T, Bs, K, dup=False, backward=False, neg=False):
    d = 64
    q, k, v = gen_inputs(seed, B, H, T, d), gen_inputs(seed + 1, B, H, T, d), gen_inputs(seed + 2, B, H, T, d)
    nb = T // Bs
    g = torch.Generator().manual_seed(seed + 7)
    idx = torch.stack([torch.stack([torch.stack([torch.randperm(nb, generator=g)[:K] if nb >= K else
                                                  torch.randint(0, nb, (K,), generator=g)
                                                  for _ in range(nb)]) for _ in range(H)]) for _ in range(B)]).int()
    if dup:       # the padding pattern of the compress kernel when Nc < K: last block repeated
        idx[..., K // 2:] = nb - 1
    if neg:       # -1 (skipped by the forward kernel, :97)
        idx[..., -3:] = -1
    scale = 1.0 / math.sqrt(d)
    o, lse = tba._topk_blocksparse_attention_fwd(q, k, v, idx, Bs, scale)
    out = dict(q=q, k=k, v=v, idx=idx, o=o, lse=lse, block=np.int32(Bs))
    if backward:
        do = gen_inputs(seed + 3, B, H, T, d)
        dq, dk, dv = tba._topk_blocksparse_attention_bwd(o, do, lse, q, k, v, idx, Bs, scale)
        out.update(do=do, dq=dq, dk=dk, dv=dv)
    save(name, **out)


# ---------------------------------------------------------------- whole module
def _patch_module(sa, tba):
    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, q, k, v, idx, block_size, scale):
            o, lse = tba._topk_blocksparse_attention_fwd(q, k, v, idx, block_size, scale)
            ctx.save_for_backward(q, k, v, o, lse, idx)
            ctx.bs, ctx.scale = block_size, scale
            return o

        @staticmethod
        def backward(ctx, do):
            q, k, v, o, lse, idx = ctx.saved_tensors
            dq, dk, dv = tba._topk_blocksparse_attention_bwd(o, do.contiguous(), lse, q, k, v, idx, ctx.bs, ctx.scale)
            return dq, dk, dv, None, None, None

    def unasserted(q, k, v, topk_idx, block_size, softmax_scale=None):
        if softmax_scale is None:
            softmax_scale = 1.0 / math.sqrt(q.shape[-1])
        return _Fn.apply(q, k, v, topk_idx, block_size, softmax_scale)

    sa.topk_blocksparse_attention = unasserted


def case_module(fat, tba, sa, RoPE2D, name, seed, B, hgrid, wgrid, views, dim, heads, backward=False):
    _patch_module(sa, tba)
    torch.manual_seed(seed)
    rope = RoPE2D(freq=100.0)
    m = sa.SparseFlashAttentionRope(dim, num_heads=heads, qkv_bias=True, proj_bias=True, qk_norm=True, rope=rope)
    # the released init leaves the gate weight at zero; give it (and the norms) content
    with torch.no_grad():
        m.gate[0].weight.normal_(0, 0.05)
        m.q_norm.weight.normal_(1, 0.1); m.q_norm.bias.normal_(0, 0.1)
        m.k_norm.weight.normal_(1, 0.1); m.k_norm.bias.normal_(0, 0.1)
    # token order of Pi3_Sparse.decode: per view, 4x4-patch block-major (pi3_sparse.py:29-45)
    ys, xs = torch.meshgrid(torch.arange(hgrid), torch.arange(wgrid), indexing="ij")
    pos = torch.stack([ys, xs], -1).view(hgrid // 4, 4, wgrid // 4, 4, 2).permute(0, 2, 1, 3, 4).reshape(-1, 2)
    xpos = pos[None].repeat(B, views, 1)
    T = xpos.shape[1]
    x = torch.randn(B, T, dim) * 1.5
    x.requires_grad_(backward)
    y = m(x, xpos=xpos)
    out = dict(x=x, xpos=xpos, y=y, heads=np.int32(heads))
    for k_, v_ in m.state_dict().items():
        out["param." + k_] = v_
    if backward:
        dy = torch.randn(B, T, dim)
        y.backward(dy)
        out.update(dy=dy, dx=x.grad)
        for k_, p in m.named_parameters():
            out["grad." + k_] = p.grad
    save(name, **out)


# ---------------------------------------------------------------- BASELINE config 1 at op level
def case_cfg1(fat, tba, name):
    """B=1, T=2048 (8 views x 256), 16 heads, d=64, seed 0, reference setting 16/16/16/32.
    q,k,v ~ N(0,1); the op pools them directly (no LN / RoPE).  Inputs are regenerated from
    the seed by the test; stored: idx, and o_c / o_s / lse subsampled."""
    torch.manual_seed(0)
    B, H, T, d, Bs, K = 1, 16, 2048, 64, 16, 32
    q, k, v = torch.randn(B, H, T, d), torch.randn(B, H, T, d), torch.randn(B, H, T, d)
    gate = torch.sigmoid(torch.randn(B, H, T, 2))
    pool = lambda z: torch.nn.functional.avg_pool1d(z.permute(0, 1, 3, 2).reshape(B * H, d, T), Bs, Bs) \
        .reshape(B, H, d, T // Bs).permute(0, 1, 3, 2).contiguous()
    q_c, k_c, v_c = pool(q), pool(k), pool(v)
    o_c, lse_c, idx, scale = fat.forward_with_topk(q_c, k_c, v_c, K)
    o_s, lse_s = tba._topk_blocksparse_attention_fwd(q, k, v, idx, Bs, scale)
    y = gate[..., 0:1] * o_c.repeat_interleave(Bs, 2) + gate[..., 1:2] * o_s
    y = y.permute(0, 2, 1, 3).reshape(B, T, H * d)
    save(name, idx=idx.to(torch.int16), o_c=o_c, lse_c=lse_c[:, :, : T // Bs], o_s_sub=o_s[:, :, ::8], lse_s=lse_s,
         y_sub=y[:, ::8], q_probe=q[0, 3, 100], gate_probe=gate[0, 5, 77])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default=None)
    a = ap.parse_args()
    fat, tba, sa, RoPE2D = _ref(a.reference)
    cases = {
        "cmp_basic":   lambda: case_cmp(fat, "cmp_basic", 10, 1, 2, 128, 128, 32, backward=True),
        "cmp_ragged":  lambda: case_cmp(fat, "cmp_ragged", 20, 1, 2, 100, 100, 32, backward=True),
        "cmp_rect":    lambda: case_cmp(fat, "cmp_rect", 25, 2, 1, 40, 150, 16),
        "cmp_short":   lambda: case_cmp(fat, "cmp_short", 30, 1, 2, 16, 16, 32),
        "cmp_ties":    lambda: case_cmp(fat, "cmp_ties", 40, 1, 2, 96, 96, 32, tie_mode=True),
        "sel_basic":   lambda: case_sel(tba, "sel_basic", 50, 1, 2, 256, 16, 8, backward=True),
        "sel_k32":     lambda: case_sel(tba, "sel_k32", 60, 1, 1, 512, 16, 32, backward=True),
        "sel_dup":     lambda: case_sel(tba, "sel_dup", 70, 1, 2, 128, 16, 8, dup=True, backward=True),
        "sel_neg":     lambda: case_sel(tba, "sel_neg", 80, 1, 1, 128, 16, 8, neg=True),
        "sel_bs64":    lambda: case_sel(tba, "sel_bs64", 90, 1, 1, 512, 64, 4, backward=True),
        "module_fwd":  lambda: case_module(fat, tba, sa, RoPE2D, "module_fwd", 100, 1, 8, 16, 4, 128, 2),
        "module_bwd":  lambda: case_module(fat, tba, sa, RoPE2D, "module_bwd", 110, 2, 8, 8, 2, 128, 2, backward=True),
        "cfg1":        lambda: case_cfg1(fat, tba, "cfg1"),
    }
    for n, fn in cases.items():
        if a.only and n not in a.only.split(","):
            continue
        t = time.time()
        fn()
        print(f"{n}: {time.time() - t:.1f}s", flush=True)


if __name__ == "__main__":
    main()
