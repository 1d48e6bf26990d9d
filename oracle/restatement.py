"""CPU restatement of Speed3R's dual-branch sparse global attention.

TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: it may be
imported by tests, by the smoke check and by the benchmark's CPU-baseline legs, never
by the product package.  It restates, in plain PyTorch on CPU (any float dtype, fp32
by default), what the reference computes with Triton kernels:

* ``pool_qkv``            – pi3/models/layers/sparse_attention.py:97-102
* ``block_positions``     – pi3/models/layers/sparse_attention.py:107-108
* ``rope2d``              – pi3/models/layers/pos_embed.py:112-159
* ``sortable_key`` / ``topk_rows`` – pi3/models/sparse_attn/topk_utils.py:19-23 and the
  composite-key streaming top-k of pi3/models/sparse_attn/flash_attention_topk.py:76-151
* ``cmp_attn_topk``       – pi3/models/sparse_attn/flash_attention_topk.py:22-152
* ``sel_attn``            – pi3/models/sparse_attn/topk_blocksparse_attention.py:35-128
* ``gated_merge``         – pi3/models/layers/sparse_attention.py:127-136
* ``key_centric_csr``     – pi3/models/sparse_attn/topk_blocksparse_attention.py:368-555
* ``module_forward``      – pi3/models/layers/sparse_attention.py:90-141

Parity pin: the reference ships no tests or golden vectors for this path.  The
restatement is pinned instead against the reference's own kernels executed on CPU
through the Triton interpreter; tests/golden/make_golden.py generates those fixtures
and tests/test_oracle_golden.py checks this file against them.

Backward passes are obtained with autograd through these functions (they are written
with differentiable gather/index ops), which equals the reference's hand-written
backward kernels up to fp rounding.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# compression (block pooling)
# --------------------------------------------------------------------------------------
def pool_qkv(qkv: torch.Tensor, num_heads: int, kernel: int = 16, stride: int = 16):
    """Mean-pool packed qkv ``[B,T,3*H*d]`` (column order (3,H,d)) over ``kernel`` tokens.

    Returns q_c, k_c, v_c each ``[B,H,Nc,d]`` with ``Nc = floor((T-kernel)/stride)+1``.
    Follows sparse_attention.py:97-102 (``F.avg_pool1d`` on the ``(b qkv h) d n`` view).
    """
    B, T, C3 = qkv.shape
    d = C3 // (3 * num_heads)
    x = qkv.reshape(B, T, 3, num_heads, d).permute(0, 2, 3, 4, 1).reshape(B * 3 * num_heads, d, T)
    x = F.avg_pool1d(x, kernel_size=kernel, stride=stride)
    Nc = x.shape[-1]
    x = x.reshape(B, 3, num_heads, d, Nc).permute(0, 2, 4, 1, 3)  # b h n qkv d
    return x[..., 0, :], x[..., 1, :], x[..., 2, :]


def pool_tokens(z: torch.Tensor, kernel: int = 16, stride: int = 16) -> torch.Tensor:
    """Mean-pool ``[B,H,T,d]`` along T (same arithmetic as ``pool_qkv`` for one tensor)."""
    B, H, T, d = z.shape
    x = z.permute(0, 1, 3, 2).reshape(B * H, d, T)
    x = F.avg_pool1d(x, kernel_size=kernel, stride=stride)
    return x.reshape(B, H, d, -1).permute(0, 1, 3, 2)


def block_positions(xpos: torch.Tensor, block: int = 16) -> torch.Tensor:
    """Truncated mean (y,x) position of each ``block`` consecutive tokens (sparse_attention.py:107-108)."""
    B, T, _ = xpos.shape
    return xpos.view(B, T // block, block, 2).float().mean(dim=2).int()


# --------------------------------------------------------------------------------------
# RoPE2D (pos_embed.py:112-159)
# --------------------------------------------------------------------------------------
def rope_tables(D: int, seq_len: int, dtype: torch.dtype, base: float = 100.0):
    """cos/sin tables ``[seq_len, D]``; the angle is rounded to ``dtype`` BEFORE cos/sin
    exactly as pos_embed.py:122-127 does."""
    inv_freq = 1.0 / (base ** (torch.arange(0, D, 2).float() / D))
    t = torch.arange(seq_len, dtype=inv_freq.dtype)
    freqs = torch.einsum("i,j->ij", t, inv_freq).to(dtype)
    freqs = torch.cat((freqs, freqs), dim=-1)
    return freqs.cos(), freqs.sin()


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope2d(tokens: torch.Tensor, positions: torch.Tensor, base: float = 100.0) -> torch.Tensor:
    """2-D rotary embedding of ``tokens [B,H,n,d]`` with integer ``positions [B,n,2]`` (y,x)."""
    D = tokens.shape[-1] // 2
    cos, sin = rope_tables(D, int(positions.max()) + 1, tokens.dtype, base)
    y, x = tokens.chunk(2, dim=-1)

    def one(t, p):
        c = F.embedding(p, cos)[:, None]
        s = F.embedding(p, sin)[:, None]
        return t * c + _rotate_half(t) * s

    return torch.cat((one(y, positions[:, :, 0].long()), one(x, positions[:, :, 1].long())), dim=-1)


# --------------------------------------------------------------------------------------
# top-k with the reference's total order
# --------------------------------------------------------------------------------------
def sortable_key(scores_fp32: np.ndarray) -> np.ndarray:
    """Order-preserving float32 -> uint32 map of topk_utils.py:19-23: flip every bit of a
    negative value, set the sign bit of a non-negative one."""
    bits = np.ascontiguousarray(scores_fp32, dtype=np.float32).view(np.uint32)
    neg = (bits & np.uint32(0x80000000)) != 0
    return np.where(neg, bits ^ np.uint32(0xFFFFFFFF), bits ^ np.uint32(0x80000000)).astype(np.uint32)


def topk_rows(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Per-row top-``k`` column indices of ``scores [..., Nq, Nc]`` (fp32), ordered by
    (value descending, column ascending), as int32 ``[..., Nq, k]``.

    flash_attention_topk.py:118-151 builds ``u64 = key<<32 | (Nc-1-col)`` for every
    column, keeps the ``k`` largest and decodes ``col = Nc-1-(u64 & 0xffffffff)``.  The
    running set starts as all-zero composites, so when ``Nc < k`` the tail decodes to
    ``Nc-1``.
    """
    s = scores.detach().to(torch.float32).cpu().numpy()
    Nc = s.shape[-1]
    key = sortable_key(s).astype(np.uint64)
    col = np.arange(Nc, dtype=np.uint64)
    comp = (key << np.uint64(32)) | (np.uint64(Nc - 1) - col)
    if Nc < k:
        pad = np.zeros(s.shape[:-1] + (k - Nc,), dtype=np.uint64)
        comp = np.concatenate([comp, pad], axis=-1)
    order = np.sort(comp, axis=-1)[..., ::-1][..., :k]
    idx = (np.uint64(Nc - 1) - (order & np.uint64(0xFFFFFFFF))).astype(np.int64)
    return torch.from_numpy(idx.astype(np.int32))


# --------------------------------------------------------------------------------------
# compression attention + top-k  (flash_attention_topk.py:22-152)
# --------------------------------------------------------------------------------------
def block_rank_scores(S: torch.Tensor, softmax_scale: float, group: int, take: int) -> torch.Tensor:
    """Selection score of key block n for every query row when the compressed keys do not map one to one
    onto selection blocks (no counterpart in the reference, whose three block sizes are equal): the softmax
    probability mass of the compressed entries whose window lies inside the block.  With windows of ``Lc``
    tokens every ``Sc`` tokens and blocks of ``Bs`` tokens those are the columns ``group*n ... group*n +
    take - 1`` with ``group = Bs/Sc`` and ``take = (Bs-Lc)/Sc + 1``.  Ranking by mass is ranking by
    ``log2 sum_j 2^(c*s_j)`` (``c = softmax_scale*log2 e``), which is what is returned: it needs no row
    normaliser, so it can be formed while the row is still streaming.  Only blocks with all ``take`` columns
    present are ranked.  ``S [..., Nq, Nc]`` raw logits -> ``[..., Nq, Nb]`` fp32."""
    Nc = S.shape[-1]
    Nb = (Nc - take) // group + 1 if Nc >= take else 0
    c = softmax_scale * 1.4426950408889634
    cols = (torch.arange(Nb)[:, None] * group + torch.arange(take)[None, :]).reshape(-1)
    g = (S.float()[..., cols] * c).reshape(*S.shape[:-1], Nb, take)
    m = g.max(dim=-1).values
    return m + torch.log2(torch.exp2(g - m[..., None]).sum(dim=-1))


def cmp_attn_topk(q_c, k_c, v_c, topk: int, softmax_scale: Optional[float] = None,
                  round_p_to: Optional[torch.dtype] = None, row_chunk: int = 4096,
                  rank_group: Optional[tuple] = None):
    """Dense non-causal attention of pooled queries over pooled keys plus the top-``topk``
    columns of the raw (unscaled) logits of every row.

    q_c ``[B,H,Nq,d]``, k_c/v_c ``[B,H,Nc,d]`` -> (o ``[B,H,Nq,d]``, lse ``[B,H,Nq]`` fp32,
    idx ``[B,H,Nq,topk]`` int32).  ``round_p_to`` mimics the kernel's cast of P to the V
    dtype before the PV product (flash_attention_topk.py:107).  ``rank_group = (group, take)``
    ranks selection blocks by ``block_rank_scores`` instead of columns by their logits.
    """
    B, H, Nq, d = q_c.shape
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    outs, lses, idxs = [], [], []
    for r0 in range(0, Nq, row_chunk):
        q = q_c[:, :, r0:r0 + row_chunk]
        S = torch.matmul(q.float(), k_c.float().transpose(-1, -2))          # raw logits, fp32
        idxs.append(topk_rows(S if rank_group is None else block_rank_scores(S, softmax_scale, *rank_group), topk))
        Ss = S * softmax_scale
        lse = torch.logsumexp(Ss, dim=-1)
        P = torch.exp(Ss - lse[..., None])
        if round_p_to is not None:
            # the kernel rounds exp(s - m) (not the normalised P); the effect on o is the same order
            P = P.to(round_p_to).float()
        outs.append(torch.matmul(P, v_c.float()).to(q_c.dtype))
        lses.append(lse)
    return torch.cat(outs, 2), torch.cat(lses, 2), torch.cat(idxs, 2)


# --------------------------------------------------------------------------------------
# selection attention  (topk_blocksparse_attention.py:35-128)
# --------------------------------------------------------------------------------------
def sel_attn(q, k, v, idx, block: int = 16, softmax_scale: Optional[float] = None,
             qblock_chunk: int = 2048):
    """Softmax attention of each query block over the multiset of its selected key blocks.

    q ``[B,H,Tq,d]``, k/v ``[B,H,Tk,d]``, idx ``[B,H,ceil(Tq/block),K]`` int32 ->
    (o ``[B,H,Tq,d]``, lse ``[B,H,Tq]`` fp32).  An entry n with ``n<0`` or
    ``n*block >= Tk`` is skipped (:97); the tail of a partial last key block is masked
    (:98); a block listed twice is counted twice.  A query row whose every entry is
    skipped gets o = 0 and lse = -inf... the kernel leaves ``lse`` at -inf and o at
    ``0 * exp(-inf - -inf)`` = NaN there; the restatement returns NaN too.
    """
    B, H, Tq, d = q.shape
    Tk = k.shape[2]
    K = idx.shape[-1]
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(d)
    nqb = (Tq + block - 1) // block
    assert idx.shape[2] == nqb
    pad_q = nqb * block - Tq
    qf = F.pad(q.float(), (0, 0, 0, pad_q)).view(B, H, nqb, block, d)
    kf, vf = k.float(), v.float()
    ar = torch.arange(block)
    outs, lses = [], []
    for m0 in range(0, nqb, qblock_chunk):
        ix = idx[:, :, m0:m0 + qblock_chunk].long()                         # [B,H,mc,K]
        mc = ix.shape[2]
        tok = ix[..., None] * block + ar                                    # [B,H,mc,K,block]
        valid_blk = (ix >= 0) & (ix * block < Tk)
        valid = valid_blk[..., None] & (tok < Tk) & (tok >= 0)
        tok_c = tok.clamp(0, Tk - 1).reshape(B, H, mc * K * block)
        gi = tok_c[..., None].expand(-1, -1, -1, d)
        kg = torch.gather(kf, 2, gi).view(B, H, mc, K * block, d)
        vg = torch.gather(vf, 2, gi).view(B, H, mc, K * block, d)
        S = torch.matmul(qf[:, :, m0:m0 + mc], kg.transpose(-1, -2)) * softmax_scale
        S = S.masked_fill(~valid.view(B, H, mc, 1, K * block), float("-inf"))
        lse = torch.logsumexp(S, dim=-1)
        P = torch.exp(S - lse[..., None])
        outs.append(torch.matmul(P, vg))
        lses.append(lse)
    o = torch.cat(outs, 2).view(B, H, nqb * block, d)[:, :, :Tq].to(q.dtype)
    lse = torch.cat(lses, 2).view(B, H, nqb * block)[:, :, :Tq]
    return o, lse


# --------------------------------------------------------------------------------------
# gated merge  (sparse_attention.py:127-136)
# --------------------------------------------------------------------------------------
def gated_merge(gate, o_c, o_s, block: int = 16):
    """``y[b,t,(h d)] = g0[b,h,t] * o_c[b,h,t//block,:] + g1[b,h,t] * o_s[b,h,t,:]``.

    gate ``[B,H,T,2]``, o_c ``[B,H,Nq,d]``, o_s ``[B,H,T,d]`` -> ``[B,T,H*d]``."""
    B, H, T, d = o_s.shape
    oc_b = o_c.repeat_interleave(block, dim=2)[:, :, :T]
    y = gate[..., 0:1] * oc_b + gate[..., 1:2] * o_s
    return y.permute(0, 2, 1, 3).reshape(B, T, H * d)


# --------------------------------------------------------------------------------------
# key-centric CSR of the index table  (topk_blocksparse_attention.py:368-555)
# --------------------------------------------------------------------------------------
def key_centric_csr(idx: torch.Tensor, num_key_blocks: int):
    """For every (b,h): ``offsets [B,H,Nkb+1]`` and the query-block ids that list each key
    block, ascending within a key block (the reference uses a stable argsort), entries
    ``<0`` or ``>= num_key_blocks`` dropped.  Returns (offsets int32, qids list-of-arrays
    flattened to ``[B,H,total]`` padded with -1)."""
    B, H, Nq, K = idx.shape
    flat = idx.reshape(B, H, Nq * K).long()
    qid = torch.arange(Nq).repeat_interleave(K)
    offs = torch.zeros(B, H, num_key_blocks + 1, dtype=torch.int32)
    total = 0
    lists = []
    for b in range(B):
        for h in range(H):
            f = flat[b, h]
            ok = (f >= 0) & (f < num_key_blocks)
            fk, fq = f[ok], qid[ok]
            order = torch.argsort(fk, stable=True)
            cnt = torch.bincount(fk, minlength=num_key_blocks)
            offs[b, h, 1:] = torch.cumsum(cnt, 0).int()
            lists.append(fq[order].int())
            total = max(total, int(ok.sum()))
    out = torch.full((B, H, total), -1, dtype=torch.int32)
    for i, l in enumerate(lists):
        out[i // H, i % H, : l.numel()] = l
    return offs, out


# --------------------------------------------------------------------------------------
# whole sparse-attention op and module
# --------------------------------------------------------------------------------------
def sparse_attention_op(q, k, v, gate, block: int = 16, topk: int = 32,
                        kernel: int = 16, stride: int = 16):
    """Op-level path used by the op sweeps: pool q,k,v directly (no LN/RoPE), compression
    attention + top-k, selection attention, gated merge.  Inputs ``[B,H,T,d]``, gate
    ``[B,H,T,2]`` (already passed through the sigmoid).  Returns (y ``[B,T,H*d]``, idx).
    Queries are pooled per selection block; keys and values with ``kernel``/``stride``.  At the reference's
    16/16/16 this is its path; for other settings the blocks are ranked by ``block_rank_scores``."""
    q_c, k_c, v_c = pool_tokens(q, block, block), pool_tokens(k, kernel, stride), pool_tokens(v, kernel, stride)
    rank_group = None
    if (kernel, stride) != (block, block):        # compressed keys and selection blocks differ: rank blocks by mass
        if block % stride or kernel > block or (block - kernel) % stride:
            raise ValueError("need stride | block and kernel = block - i*stride")
        rank_group = (block // stride, (block - kernel) // stride + 1)
    o_c, _, idx = cmp_attn_topk(q_c, k_c, v_c, topk, rank_group=rank_group)
    o_s, _ = sel_attn(q, k, v, idx, block)
    return gated_merge(gate, o_c, o_s, block), idx


def layer_norm_heads(x, weight, bias, eps=1e-5):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps)


def qkv_prologue(qkv: torch.Tensor, num_heads: int, block: int = 16, xpos: Optional[torch.Tensor] = None,
                 q_norm=None, k_norm=None, rope_base: float = 100.0):
    """The steps between the qkv projection and the two attention calls (sparse_attention.py:95-123)
    as one function: ``qkv [B,T,3*H*d]`` -> ``(q, k, v [B,H,T,d], q_c, k_c, v_c [B,H,T/block,d])``.
    ``q_norm``/``k_norm`` are ``(weight, bias)`` pairs or None; the pooled q and k get the same norm and
    the rotary embedding at the truncated mean position of their block."""
    B, T, _ = qkv.shape
    H = num_heads
    d = qkv.shape[-1] // (3 * H)
    q_c, k_c, v_c = pool_qkv(qkv, H, block, block)
    full = qkv.reshape(B, T, 3, H, d).transpose(1, 3)
    q, k, v = full[:, :, 0], full[:, :, 1], full[:, :, 2]
    if q_norm is not None:
        q_c, q = (layer_norm_heads(t, q_norm[0], q_norm[1]).to(v.dtype) for t in (q_c, q))
        k_c, k = (layer_norm_heads(t, k_norm[0], k_norm[1]).to(v.dtype) for t in (k_c, k))
    if xpos is not None:
        pc = block_positions(xpos, block)
        q_c, k_c = rope2d(q_c, pc, rope_base), rope2d(k_c, pc, rope_base)
        q, k = rope2d(q, xpos, rope_base), rope2d(k, xpos, rope_base)
    return q, k, v, q_c, k_c, v_c


def module_forward(params: dict, x: torch.Tensor, xpos: Optional[torch.Tensor], num_heads: int,
                   block_size: int = 4, topk: int = 32, rope_base: float = 100.0,
                   return_aux: bool = False, idx_override: Optional[torch.Tensor] = None):
    """Restatement of ``SparseFlashAttentionRope.forward`` (sparse_attention.py:90-141).

    ``params`` uses the module's state-dict keys (``qkv.weight`` ... ``gate.0.bias``).
    Runs in the dtype of ``x`` (fp32 for the oracle).  ``idx_override`` replaces the selected
    block table (used to compare a bf16 run, whose near-tie selections may differ, on equal terms)."""
    B, T, C = x.shape
    H = num_heads
    d = C // H
    Bs = block_size ** 2
    qkv = F.linear(x, params["qkv.weight"], params.get("qkv.bias"))
    gate = torch.sigmoid(F.linear(x, params["gate.0.weight"], params["gate.0.bias"]))
    gate = gate.view(B, T, H, 2).permute(0, 2, 1, 3)
    q_c, k_c, v_c = pool_qkv(qkv, H, Bs, Bs)
    has_norm = "q_norm.weight" in params
    if has_norm:
        q_c = layer_norm_heads(q_c, params["q_norm.weight"], params["q_norm.bias"]).to(v_c.dtype)
        k_c = layer_norm_heads(k_c, params["k_norm.weight"], params["k_norm.bias"]).to(v_c.dtype)
    if xpos is not None:
        pc = block_positions(xpos, Bs)
        q_c, k_c = rope2d(q_c, pc, rope_base), rope2d(k_c, pc, rope_base)
    o_c, _, idx = cmp_attn_topk(q_c, k_c, v_c, topk)
    if idx_override is not None:
        idx = idx_override
    qkv_full = qkv.reshape(B, T, 3, H, d).transpose(1, 3)
    q, k, v = qkv_full[:, :, 0], qkv_full[:, :, 1], qkv_full[:, :, 2]
    if has_norm:
        q = layer_norm_heads(q, params["q_norm.weight"], params["q_norm.bias"]).to(v.dtype)
        k = layer_norm_heads(k, params["k_norm.weight"], params["k_norm.bias"]).to(v.dtype)
    if xpos is not None:
        q, k = rope2d(q, xpos, rope_base), rope2d(k, xpos, rope_base)
    o_s, _ = sel_attn(q, k, v, idx, Bs)
    y = gated_merge(gate, o_c, o_s, Bs)
    out = F.linear(y, params["proj.weight"], params.get("proj.bias"))
    if return_aux:
        return out, dict(idx=idx, o_c=o_c, o_s=o_s, y=y, q=q, k=k, v=v, q_c=q_c, k_c=k_c, v_c=v_c, gate=gate)
    return out
