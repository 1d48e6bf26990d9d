"""Thin ``torch.library`` layer over the C-ABI kernels.

Public functions mirror the reference's op signatures:

* ``flash_attn_topk_func(q_c, k_c, v_c, topk_val, bias=None, causal=False, softmax_scale=None)``
  -> ``(o_c, idx)``      (pi3/models/sparse_attn/flash_attention_topk.py:633-668)
* ``topk_blocksparse_attention(q, k, v, topk_idx, block_size, softmax_scale=None)`` -> ``o``
  (pi3/models/sparse_attn/topk_blocksparse_attention.py:1093-1121)

plus the pieces the reference leaves to eager PyTorch (sparse_attention.py:97-102, 127-136):

* ``pool_tokens(x, kernel, stride)``: mean pooling along the sequence
* ``sel_attn_merge(q, k, v, idx, gate, o_c, block_size)``: selection attention with the gated
  merge fused, returning ``[B,T,H*d]``

This layer owns allocation, argument checks and autograd wiring only; all arithmetic runs in the
CUDA library.  CPU tensors, fp32/fp16 inputs and a missing library raise — there is no fallback.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

_BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: Tensor, name: str, dtype=_BF16, contiguous=True) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: the speed3r_b200 kernels have no CPU path")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _ptr(t: Optional[Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


# ------------------------------------------------------------------------------------------------
# raw kernels as custom ops
# ------------------------------------------------------------------------------------------------
@torch.library.custom_op("speed3r_b200::pool_fwd", mutates_args=())
def _pool_fwd(x: Tensor, kernel: int, stride: int) -> Tensor:
    _need(x, "x", contiguous=False)
    B, H, T, d = x.shape
    if x.stride(3) != 1:
        raise RuntimeError("pool: the channel dimension must have unit stride")
    Nc = (T - kernel) // stride + 1
    out = torch.empty(B, H, Nc, d, device=x.device, dtype=x.dtype)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().s3r_pool_fwd(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), out.data_ptr(),
                                            B, H, T, d, kernel, stride, _stream()), "s3r_pool_fwd")
    return out


@_pool_fwd.register_fake
def _(x, kernel, stride):
    B, H, T, d = x.shape
    return x.new_empty(B, H, (T - kernel) // stride + 1, d)


def qkv_prologue(qkv: Tensor, num_heads: int, block: int, pos: Optional[Tensor] = None,
                 cos: Optional[Tensor] = None, sin: Optional[Tensor] = None,
                 q_norm: Optional[Tuple[Tensor, Tensor, float]] = None,
                 k_norm: Optional[Tuple[Tensor, Tensor, float]] = None):
    """Everything between the qkv projection and the two attention calls of the module
    (pi3/models/layers/sparse_attention.py:95-123) in one kernel, forward only:
    ``qkv [B,N,3*H*d]`` -> ``(q, k, v [B,H,N,d], q_c, k_c, v_c [B,H,N/block,d])`` with the per-head
    LayerNorm of q and k (``(weight, bias, eps)`` or None), the 2-D rotary embedding at ``pos
    [B,N,2]`` (``cos``/``sin`` = the bf16 tables RoPE2D caches) and, for the pooled tensors, at each
    block's truncated mean position."""
    _need(qkv, "qkv")
    if qkv.requires_grad and torch.is_grad_enabled():
        raise RuntimeError("qkv_prologue is forward-only; run the separate steps when gradients are needed")
    B, N, C3 = qkv.shape[0], qkv.shape[1], qkv.numel() // (qkv.shape[0] * qkv.shape[1])
    d = C3 // (3 * num_heads)
    if C3 != 3 * num_heads * d or N % block:
        raise RuntimeError(f"qkv_prologue: qkv {tuple(qkv.shape)} does not split into 3 x {num_heads} heads, "
                           f"or N={N} is not a multiple of the block {block}")
    if (q_norm is None) != (k_norm is None):
        raise RuntimeError("qkv_prologue: q_norm and k_norm come together or not at all")
    dev = qkv.device
    f32 = lambda t: t.detach().to(device=dev, dtype=torch.float32).contiguous()
    qw = qb = kw = kb = None
    eps = 1e-5
    if q_norm is not None:
        if abs(q_norm[2] - k_norm[2]) > 0:
            raise RuntimeError("qkv_prologue: q_norm and k_norm must share eps")
        qw, qb, kw, kb, eps = f32(q_norm[0]), f32(q_norm[1]), f32(k_norm[0]), f32(k_norm[1]), float(q_norm[2])
    rows = 0
    if pos is not None:
        _need(cos, "cos")
        _need(sin, "sin")
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != d // 2:
            raise RuntimeError(f"qkv_prologue: cos/sin tables must be [rows,{d // 2}]")
        if tuple(pos.shape) != (B, N, 2) or pos.device != dev:
            raise RuntimeError(f"qkv_prologue: pos must be [B,N,2] = {(B, N, 2)} on {dev}")
        pos = pos.to(torch.int64).contiguous()
        rows = cos.shape[0]
    mk = lambda n: torch.empty(B, num_heads, n, d, device=dev, dtype=qkv.dtype)
    q, k, v = mk(N), mk(N), mk(N)
    q_c, k_c, v_c = mk(N // block), mk(N // block), mk(N // block)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().s3r_qkv_prologue_fwd(
            qkv.data_ptr(), _ptr(pos), _ptr(cos) if pos is not None else 0, _ptr(sin) if pos is not None else 0, rows,
            _ptr(qw), _ptr(qb), _ptr(kw), _ptr(kb), eps, q.data_ptr(), k.data_ptr(), v.data_ptr(),
            q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), B, num_heads, N, d, block, _stream()),
            "s3r_qkv_prologue_fwd")
    return q, k, v, q_c, k_c, v_c


@torch.library.custom_op("speed3r_b200::pool_bwd", mutates_args=())
def _pool_bwd(d_out: Tensor, T: int, kernel: int, stride: int) -> Tensor:
    _need(d_out, "d_out")
    B, H, Nc, d = d_out.shape
    d_in = torch.empty(B, H, T, d, device=d_out.device, dtype=d_out.dtype)
    with torch.cuda.device(d_out.device):
        _lib.check(_lib.load().s3r_pool_bwd(d_out.data_ptr(), d_in.data_ptr(), H * T * d, T * d, d, B, H, T, d,
                                            kernel, stride, 0, _stream()), "s3r_pool_bwd")
    return d_in


@_pool_bwd.register_fake
def _(d_out, T, kernel, stride):
    B, H, Nc, d = d_out.shape
    return d_out.new_empty(B, H, T, d)


@torch.library.custom_op("speed3r_b200::cmp_attn_topk_fwd", mutates_args=())
def _cmp_fwd(q_c: Tensor, k_c: Tensor, v_c: Tensor, topk: int, scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    for n, t in (("q_c", q_c), ("k_c", k_c), ("v_c", v_c)):
        _need(t, n)
    B, H, Nq, d = q_c.shape
    Nc = k_c.shape[2]
    if k_c.shape != (B, H, Nc, d) or v_c.shape != (B, H, Nc, d):
        raise RuntimeError(f"k_c/v_c shape mismatch: {tuple(k_c.shape)} {tuple(v_c.shape)} vs B={B} H={H} d={d}")
    o = torch.empty_like(q_c)
    lse = torch.empty(B, H, Nq, device=q_c.device, dtype=torch.float32)
    idx = torch.empty(B, H, Nq, topk, device=q_c.device, dtype=torch.int32)
    with torch.cuda.device(q_c.device):
        _lib.check(_lib.load().s3r_cmp_attn_topk_fwd(q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), o.data_ptr(),
                                                     lse.data_ptr(), idx.data_ptr(), B, H, Nq, Nc, d, topk, scale,
                                                     _stream()), "s3r_cmp_attn_topk_fwd")
    return o, lse, idx


@_cmp_fwd.register_fake
def _(q_c, k_c, v_c, topk, scale):
    B, H, Nq, d = q_c.shape
    return (torch.empty_like(q_c), q_c.new_empty(B, H, Nq, dtype=torch.float32),
            q_c.new_empty(B, H, Nq, topk, dtype=torch.int32))


@torch.library.custom_op("speed3r_b200::cmp_attn_blocktopk_fwd", mutates_args=())
def _cmp_block_fwd(q_c: Tensor, k_c: Tensor, v_c: Tensor, topk: int, scale: float, group: int,
                   take: int) -> Tuple[Tensor, Tensor, Tensor]:
    for n, t in (("q_c", q_c), ("k_c", k_c), ("v_c", v_c)):
        _need(t, n)
    B, H, Nq, d = q_c.shape
    Nc = k_c.shape[2]
    if k_c.shape != (B, H, Nc, d) or v_c.shape != (B, H, Nc, d):
        raise RuntimeError(f"k_c/v_c shape mismatch: {tuple(k_c.shape)} {tuple(v_c.shape)} vs B={B} H={H} d={d}")
    o = torch.empty_like(q_c)
    lse = torch.empty(B, H, Nq, device=q_c.device, dtype=torch.float32)
    idx = torch.empty(B, H, Nq, topk, device=q_c.device, dtype=torch.int32)
    with torch.cuda.device(q_c.device):
        _lib.check(_lib.load().s3r_cmp_attn_blocktopk_fwd(q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), o.data_ptr(),
                                                          lse.data_ptr(), idx.data_ptr(), B, H, Nq, Nc, d, topk, scale,
                                                          group, take, _stream()), "s3r_cmp_attn_blocktopk_fwd")
    return o, lse, idx


@_cmp_block_fwd.register_fake
def _(q_c, k_c, v_c, topk, scale, group, take):
    B, H, Nq, d = q_c.shape
    return (torch.empty_like(q_c), q_c.new_empty(B, H, Nq, dtype=torch.float32),
            q_c.new_empty(B, H, Nq, topk, dtype=torch.int32))


@torch.library.custom_op("speed3r_b200::cmp_attn_bwd", mutates_args=())
def _cmp_bwd(q_c: Tensor, k_c: Tensor, v_c: Tensor, o_c: Tensor, lse: Tensor, do_c: Tensor,
             scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    for n, t in (("q_c", q_c), ("k_c", k_c), ("v_c", v_c), ("o_c", o_c), ("do_c", do_c)):
        _need(t, n)
    _need(lse, "lse", torch.float32)
    B, H, Nq, d = q_c.shape
    Nc = k_c.shape[2]
    dq, dk, dv = torch.empty_like(q_c), torch.empty_like(k_c), torch.empty_like(v_c)
    delta = torch.empty_like(lse)
    with torch.cuda.device(q_c.device):
        _lib.check(_lib.load().s3r_cmp_attn_bwd(q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), o_c.data_ptr(),
                                                lse.data_ptr(), do_c.data_ptr(), delta.data_ptr(), dq.data_ptr(),
                                                dk.data_ptr(), dv.data_ptr(), B, H, Nq, Nc, d, scale, _stream()),
                   "s3r_cmp_attn_bwd")
    return dq, dk, dv


@_cmp_bwd.register_fake
def _(q_c, k_c, v_c, o_c, lse, do_c, scale):
    return torch.empty_like(q_c), torch.empty_like(k_c), torch.empty_like(v_c)


def _gate_strides(gate: Tensor):
    if gate.stride(3) != 1:
        raise RuntimeError("gate: the last dimension (g0,g1) must have unit stride")
    return gate.stride(0), gate.stride(1), gate.stride(2)


@torch.library.custom_op("speed3r_b200::sel_attn_fwd", mutates_args=())
def _sel_fwd(q: Tensor, k: Tensor, v: Tensor, idx: Tensor, gate: Optional[Tensor], o_c: Optional[Tensor],
             block: int, scale: float, want_o: bool, want_lse: bool, kv_chunks: int) -> Tuple[Tensor, Tensor, Tensor]:
    """Returns (o_s, lse_s, y); tensors not asked for come back with zero elements."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _need(t, n)
    _need(idx, "topk_idx", torch.int32)
    B, H, Tq, d = q.shape
    if kv_chunks == 1:
        Tk, chunk_stride = k.shape[2], 0
        if k.shape != (B, H, Tk, d) or v.shape != k.shape:
            raise RuntimeError("k/v must be [B,H,Tk,d]")
    else:                                # [chunks, B, H, Tk/chunks, d] as an all-gather leaves it
        if k.dim() != 5 or k.shape[0] != kv_chunks or v.shape != k.shape:
            raise RuntimeError("chunked k/v must be [chunks,B,H,Tk/chunks,d]")
        Tk, chunk_stride = k.shape[3] * kv_chunks, k.stride(0)
    K = idx.shape[-1]
    nqb = (Tq + block - 1) // block
    if tuple(idx.shape) != (B, H, nqb, K):
        raise RuntimeError(f"topk_idx must be [B,H,ceil(Tq/block),K] = {(B, H, nqb, K)}, got {tuple(idx.shape)}")
    merge = gate is not None
    if merge:
        _need(gate, "gate", contiguous=False)
        _need(o_c, "o_c")
        if tuple(gate.shape) != (B, H, Tq, 2) or tuple(o_c.shape) != (B, H, nqb, d):
            raise RuntimeError("gate must be [B,H,Tq,2] and o_c [B,H,ceil(Tq/block),d]")
        gs = _gate_strides(gate)
    else:
        gs = (0, 0, 0)
    dev = q.device
    o_s = torch.empty(B, H, Tq, d, device=dev, dtype=q.dtype) if want_o else q.new_empty(0)
    lse = torch.empty(B, H, Tq, device=dev, dtype=torch.float32) if want_lse else q.new_empty(0, dtype=torch.float32)
    y = torch.empty(B, Tq, H * d, device=dev, dtype=q.dtype) if merge else q.new_empty(0)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().s3r_sel_attn_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_chunks, chunk_stride, idx.data_ptr(),
            o_s.data_ptr() if want_o else 0, lse.data_ptr() if want_lse else 0,
            _ptr(gate), gs[0], gs[1], gs[2], _ptr(o_c), y.data_ptr() if merge else 0,
            B, H, Tq, Tk, d, block, K, scale, _stream()), "s3r_sel_attn_fwd")
    return o_s, lse, y


@_sel_fwd.register_fake
def _(q, k, v, idx, gate, o_c, block, scale, want_o, want_lse, kv_chunks):
    B, H, Tq, d = q.shape
    return (q.new_empty(B, H, Tq, d) if want_o else q.new_empty(0),
            q.new_empty(B, H, Tq, dtype=torch.float32) if want_lse else q.new_empty(0, dtype=torch.float32),
            q.new_empty(B, Tq, H * d) if gate is not None else q.new_empty(0))


@torch.library.custom_op("speed3r_b200::build_key_csr", mutates_args=())
def build_key_csr(idx: Tensor, num_key_blocks: int) -> Tuple[Tensor, Tensor]:
    """Key-centric CSR of the selection table: (offsets [B,H,Nkb+1], qids [B,H,Nq*K]) int32."""
    _need(idx, "topk_idx", torch.int32)
    B, H, Nq, K = idx.shape
    lib = _lib.load()
    offsets = torch.empty(B, H, num_key_blocks + 1, device=idx.device, dtype=torch.int32)
    qids = torch.full((B, H, Nq * K), -1, device=idx.device, dtype=torch.int32)
    nbytes = lib.s3r_csr_workspace_bytes(B, H, Nq, K, num_key_blocks)
    ws = torch.empty(nbytes, device=idx.device, dtype=torch.uint8)
    with torch.cuda.device(idx.device):
        _lib.check(lib.s3r_build_key_csr(idx.data_ptr(), offsets.data_ptr(), qids.data_ptr(), B, H, Nq, K,
                                         num_key_blocks, ws.data_ptr(), nbytes, _stream()), "s3r_build_key_csr")
    return offsets, qids


@build_key_csr.register_fake
def _(idx, num_key_blocks):
    B, H, Nq, K = idx.shape
    return idx.new_empty(B, H, num_key_blocks + 1), idx.new_empty(B, H, Nq * K)


@torch.library.custom_op("speed3r_b200::sel_attn_bwd", mutates_args=())
def _sel_bwd(q: Tensor, k: Tensor, v: Tensor, idx: Tensor, lse: Tensor, delta: Tensor, do_s: Tensor,
             block: int, scale: float) -> Tuple[Tensor, Tensor, Tensor]:
    for n, t in (("q", q), ("k", k), ("v", v), ("do_s", do_s)):
        _need(t, n)
    B, H, Tq, d = q.shape
    Tk = k.shape[2]
    K = idx.shape[-1]
    offsets, qids = build_key_csr(idx, (Tk + block - 1) // block)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().s3r_sel_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), idx.data_ptr(), offsets.data_ptr(), qids.data_ptr(),
            lse.data_ptr(), delta.data_ptr(), do_s.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            B, H, Tq, Tk, d, block, K, scale, _stream()), "s3r_sel_attn_bwd")
    return dq, dk, dv


@_sel_bwd.register_fake
def _(q, k, v, idx, lse, delta, do_s, block, scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


@torch.library.custom_op("speed3r_b200::delta", mutates_args=())
def _delta(o: Tensor, d_o: Tensor) -> Tensor:
    _need(o, "o")
    _need(d_o, "do")
    out = torch.empty(o.shape[:-1], device=o.device, dtype=torch.float32)
    with torch.cuda.device(o.device):
        _lib.check(_lib.load().s3r_delta(o.data_ptr(), d_o.data_ptr(), out.data_ptr(), out.numel(), o.shape[-1],
                                         _stream()), "s3r_delta")
    return out


@_delta.register_fake
def _(o, d_o):
    return o.new_empty(o.shape[:-1], dtype=torch.float32)


@torch.library.custom_op("speed3r_b200::merge_bwd", mutates_args=())
def _merge_bwd(dy: Tensor, gate: Tensor, o_c: Tensor, o_s: Tensor, block: int) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    _need(dy, "dy")
    _need(gate, "gate", contiguous=False)
    B, H, Tq, d = o_s.shape
    nqb = o_c.shape[2]
    do_s = torch.empty_like(o_s)
    dgate = torch.empty(B, H, Tq, 2, device=dy.device, dtype=torch.float32)
    do_c = torch.empty_like(o_c)
    delta = torch.empty(B, H, Tq, device=dy.device, dtype=torch.float32)
    gs = _gate_strides(gate)
    with torch.cuda.device(dy.device):
        _lib.check(_lib.load().s3r_merge_bwd(dy.data_ptr(), gate.data_ptr(), gs[0], gs[1], gs[2], o_c.data_ptr(),
                                             o_s.data_ptr(), do_s.data_ptr(), dgate.data_ptr(), do_c.data_ptr(),
                                             delta.data_ptr(), B, H, Tq, d, block, _stream()), "s3r_merge_bwd")
    return do_s, dgate, do_c, delta


@_merge_bwd.register_fake
def _(dy, gate, o_c, o_s, block):
    B, H, Tq, d = o_s.shape
    return (torch.empty_like(o_s), o_s.new_empty(B, H, Tq, 2, dtype=torch.float32), torch.empty_like(o_c),
            o_s.new_empty(B, H, Tq, dtype=torch.float32))


# ------------------------------------------------------------------------------------------------
# autograd wiring
# ------------------------------------------------------------------------------------------------
class _Pool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride):
        ctx.T, ctx.kernel, ctx.stride = x.shape[2], kernel, stride
        return _pool_fwd(x, kernel, stride)

    @staticmethod
    def backward(ctx, d_out):
        return _pool_bwd(d_out.contiguous(), ctx.T, ctx.kernel, ctx.stride), None, None


def pool_tokens(x: Tensor, kernel: int = 16, stride: int = 16) -> Tensor:
    """Mean over ``kernel`` consecutive tokens every ``stride`` tokens of ``x [B,H,T,d]`` (any
    batch/head/token strides) -> ``[B,H,Nc,d]``.  sparse_attention.py:97-102 for one of q/k/v."""
    return _Pool.apply(x, kernel, stride)


class _FlashAttnTopk(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, topk, scale):
        q, k, v = [x if x.is_contiguous() else x.contiguous() for x in (q, k, v)]
        o, lse, idx = _cmp_fwd(q, k, v, topk, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        ctx.mark_non_differentiable(idx)
        return o, idx

    @staticmethod
    def backward(ctx, do, _didx):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = _cmp_bwd(q, k, v, o, lse, do.contiguous(), ctx.scale)
        return dq, dk, dv, None, None


class _FlashAttnBlockTopk(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, topk, scale, group, take):
        q, k, v = [x if x.is_contiguous() else x.contiguous() for x in (q, k, v)]
        o, lse, idx = _cmp_block_fwd(q, k, v, topk, scale, group, take)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        ctx.mark_non_differentiable(idx)
        return o, idx

    @staticmethod
    def backward(ctx, do, _didx):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = _cmp_bwd(q, k, v, o, lse, do.contiguous(), ctx.scale)
        return dq, dk, dv, None, None, None, None


def flash_attn_blocktopk_func(q, k, v, topk_val, group, take, softmax_scale=None):
    """Compression attention whose table ranks selection BLOCKS by the softmax mass of their own compressed
    keys (columns ``group*n .. group*n+take-1``): for settings where compressed keys are finer than selection
    blocks.  Returns ``(o, idx)`` like ``flash_attn_topk_func``; ``idx`` holds block numbers."""
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    return _FlashAttnBlockTopk.apply(q, k, v, int(topk_val), float(softmax_scale), int(group), int(take))


def sparse_attention_op(q, k, v, gate, block_size=16, topk=32, kernel=16, stride=16):
    """The whole op on ``q,k,v [B,H,T,d]`` and ``gate [B,H,T,2]``: queries pooled per selection block
    (``block_size`` tokens), keys and values pooled with ``kernel``/``stride``, compression attention with the
    fused table, selection attention over the table's blocks, gated merge.  At 16/16/16 this is the
    reference's path (``sparse_attention.py:95-136`` without the norms and rotary embedding); when compressed
    keys are finer than selection blocks (e.g. kernel 32, stride 16, blocks of 64) the blocks are ranked by
    probability mass.  Returns ``(y [B,T,H*d], idx)``."""
    q_c = pool_tokens(q, block_size, block_size)
    k_c, v_c = pool_tokens(k, kernel, stride), pool_tokens(v, kernel, stride)
    if (kernel, stride) == (block_size, block_size):
        o_c, idx = flash_attn_topk_func(q_c, k_c, v_c, topk)
    else:
        if block_size % stride or kernel > block_size or (block_size - kernel) % stride:
            raise RuntimeError("need stride | block_size and kernel = block_size - i*stride")
        o_c, idx = flash_attn_blocktopk_func(q_c, k_c, v_c, topk, block_size // stride,
                                             (block_size - kernel) // stride + 1)
    return sel_attn_merge(q, k, v, idx, gate, o_c, block_size), idx


def flash_attn_topk_func(q, k, v, topk_val, bias=None, causal=False, softmax_scale=None):
    """Compression attention with fused top-k selection; drop-in for the reference's
    ``flash_attn_topk_func`` (flash_attention_topk.py:633-668).  Inputs ``[B,H,n,d]`` bf16."""
    assert bias is None, "bias is not supported (the reference ignores it as well)"
    assert not causal, "the sparse global attention is bidirectional; causal is not implemented"
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    return _FlashAttnTopk.apply(q, k, v, int(topk_val), float(softmax_scale))


class _TopkBlockSparse(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, idx, block, scale):
        need_grad = any(ctx.needs_input_grad[:3])
        o, lse, _ = _sel_fwd(q, k, v, idx, None, None, block, scale, True, need_grad, 1)
        if need_grad:
            ctx.save_for_backward(q, k, v, o, lse, idx)
        ctx.block, ctx.scale = block, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, idx = ctx.saved_tensors
        do = do.contiguous()
        dq, dk, dv = _sel_bwd(q, k, v, idx, lse, _delta(o, do), do, ctx.block, ctx.scale)
        return dq, dk, dv, None, None, None


def topk_blocksparse_attention(q, k, v, topk_idx, block_size, softmax_scale=None):
    """Block-sparse selection attention; drop-in for the reference's ``topk_blocksparse_attention``
    (topk_blocksparse_attention.py:1093-1121).  q,k,v ``[B,H,T,d]`` bf16 contiguous, ``topk_idx``
    ``[B,H,T/block,K]`` int32."""
    assert q.dtype == torch.bfloat16, "bf16 only"
    assert q.dtype == k.dtype and k.dtype == v.dtype
    assert topk_idx.dtype == torch.int32
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    return _TopkBlockSparse.apply(q, k, v, topk_idx, int(block_size), float(softmax_scale))


class _SelMerge(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, idx, gate, o_c, block, scale):
        need_grad = any(ctx.needs_input_grad[i] for i in (0, 1, 2, 4, 5))
        o_s, lse, y = _sel_fwd(q, k, v, idx, gate, o_c, block, scale, need_grad, need_grad, 1)
        if need_grad:
            ctx.save_for_backward(q, k, v, idx, gate, o_c, o_s, lse)
        ctx.block, ctx.scale = block, scale
        return y

    @staticmethod
    def backward(ctx, dy):
        q, k, v, idx, gate, o_c, o_s, lse = ctx.saved_tensors
        do_s, dgate, do_c, delta = _merge_bwd(dy.contiguous(), gate, o_c, o_s, ctx.block)
        dq, dk, dv = _sel_bwd(q, k, v, idx, lse, delta, do_s, ctx.block, ctx.scale)
        return dq, dk, dv, None, dgate.to(gate.dtype), do_c, None, None


def sel_attn_merge(q, k, v, topk_idx, gate, o_c, block_size, softmax_scale=None):
    """Selection attention with the gated merge fused into its epilogue:
    ``y[b,t,(h d)] = gate[b,h,t,0] * o_c[b,h,t//block] + gate[b,h,t,1] * sel_attn(q,k,v)[b,h,t]``
    (topk_blocksparse_attention.py:35-128 + sparse_attention.py:127-136).  ``gate [B,H,T,2]`` may
    be a strided view of the ``[B,T,2H]`` projection."""
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    return _SelMerge.apply(q, k, v, topk_idx, gate, o_c, int(block_size), float(softmax_scale))


def sel_attn_merge_chunked(q, k_chunks, v_chunks, topk_idx, gate, o_c, block_size, softmax_scale=None):
    """Forward-only form of ``sel_attn_merge`` for sequence-partitioned inference: the keys and
    values are the all-gathered ``[G,B,H,Tk/G,d]`` chunks (rank order = sequence order), read in
    place; ``q``, ``gate``, ``o_c`` and ``topk_idx`` are the local query rows; ``topk_idx`` holds
    GLOBAL key-block numbers."""
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    with torch.no_grad():
        _, _, y = _sel_fwd(q, k_chunks, v_chunks, topk_idx, gate, o_c, int(block_size), float(softmax_scale),
                           False, False, int(k_chunks.shape[0]))
    return y
