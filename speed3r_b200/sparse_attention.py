"""Drop-in replacement for the reference's global-attention module.

``SparseFlashAttentionRope`` keeps the constructor signature, sub-module names (``qkv``, ``proj``,
``q_norm``, ``k_norm``, ``gate`` = Sequential(Linear, Sigmoid)), attributes and ``forward(x,
attn_bias=None, xpos=None)`` of pi3/models/layers/sparse_attention.py:60-141, so a checkpoint of
the reference loads unchanged and ``BlockRope(attn_class=SparseFlashAttentionRope)`` works
(pi3/models/layers/block.py:282-312).  The projections stay PyTorch (cuBLAS) code; pooling, the compression attention with its top-k
selection, the selection attention and the gated merge run in the CUDA library (speed3r_b200.ops).
Without gradients the LayerNorms, the rotary embedding, the pooling and the q/k/v split run as one
library kernel as well (``ops.qkv_prologue``); with gradients they stay PyTorch code around the
differentiable ops.

The reference's literals (pooling 16/16, top-k 32) are keyword arguments here with the same
defaults.
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch
from torch import Tensor, nn

from . import ops


class _TableRows:
    """How many rows the rotary cos/sin tables need for a position tensor, without reading
    ``positions.max()`` back on every call.

    Row r of the tables depends on r alone (pos_embed.py:119-129), so a table that is longer than
    needed gives bit-identical results; only a table that is too SHORT is an error.  The size is
    therefore grow-only, and the maximum of a position tensor is read back once per tensor
    *object*: the entry is keyed on the storage-owning base tensor through a weak reference (all
    the reshaped views the decode loop passes down share one base) together with its in-place
    version counter, and is dropped when that tensor dies.  A new tensor that happens to reuse
    the address of an old one is a new object and is measured again."""

    def __init__(self, min_rows: int = 64):
        self.rows = min_rows
        self._seen = {}

    def __call__(self, positions: Tensor) -> int:
        base = positions._base if positions._base is not None else positions
        key = id(base)
        hit = self._seen.get(key)
        if hit is not None and hit[0]() is base and hit[1] == base._version:
            return self.rows
        need = int(base.max()) + 1 if base.numel() else 1        # one read-back per position tensor
        self.rows = max(self.rows, need)
        seen = self._seen
        self._seen[key] = (weakref.ref(base, lambda _r, k=key: seen.pop(k, None)), base._version)
        return self.rows


def rope_tables(rope, D: int, rows: int, device, dtype):
    """cos/sin tables ``[rows, 2*(D/2)]`` with the reference's arithmetic (pos_embed.py:119-129: the
    angle is rounded to ``dtype`` before cos/sin).  ``rope`` is this package's ``RoPE2D`` or the
    reference's: for the latter its own ``get_cos_sin`` builds (and caches) the tables."""
    if hasattr(rope, "_cos_sin"):
        return rope._cos_sin(D, rows, device, dtype)
    return rope.get_cos_sin(D, rows, device, dtype)


def _is_rope2d(rope) -> bool:
    """This package's RoPE2D or the reference's pure-PyTorch one (same attributes and table builder)."""
    return isinstance(rope, RoPE2D) or (hasattr(rope, "base") and hasattr(rope, "F0") and
                                        callable(getattr(rope, "get_cos_sin", None)))


class RoPE2D(nn.Module):
    """2-D rotary embedding with the arithmetic of pi3/models/layers/pos_embed.py:112-159 (the
    angle table is rounded to the activation dtype before cos/sin).  Unlike the reference it does
    not read ``positions.max()`` back on every call: the tables only ever grow, and a position
    tensor is measured once (see ``_TableRows``)."""

    def __init__(self, freq: float = 100.0, F0: float = 1.0):
        super().__init__()
        self.base = freq
        self.F0 = F0
        self._tables = {}
        self._rows = _TableRows()

    def _cos_sin(self, D, seq_len, device, dtype):
        key = (D, seq_len, device, dtype)
        if key not in self._tables:
            inv_freq = 1.0 / (self.base ** (torch.arange(0, D, 2).float().to(device) / D))
            t = torch.arange(seq_len, device=device, dtype=inv_freq.dtype)
            freqs = torch.einsum("i,j->ij", t, inv_freq).to(dtype)
            freqs = torch.cat((freqs, freqs), dim=-1)
            self._tables[key] = (freqs.cos(), freqs.sin())
        return self._tables[key]

    get_cos_sin = _cos_sin          # the reference's name for the same builder

    def _seq_len(self, positions: Tensor) -> int:
        return self._rows(positions)

    @staticmethod
    def _rope1d(tokens, pos1d, cos, sin):
        cos = torch.nn.functional.embedding(pos1d, cos)[:, None, :, :]
        sin = torch.nn.functional.embedding(pos1d, sin)[:, None, :, :]
        x1, x2 = tokens[..., : tokens.shape[-1] // 2], tokens[..., tokens.shape[-1] // 2:]
        return tokens * cos + torch.cat((-x2, x1), dim=-1) * sin

    def forward(self, tokens: Tensor, positions: Tensor, seq_len: Optional[int] = None) -> Tensor:
        D = tokens.size(3) // 2
        if seq_len is None:
            seq_len = self._seq_len(positions)
        cos, sin = self._cos_sin(D, seq_len, tokens.device, tokens.dtype)
        y, x = tokens.chunk(2, dim=-1)
        y = self._rope1d(y, positions[:, :, 0], cos, sin)
        x = self._rope1d(x, positions[:, :, 1], cos, sin)
        return torch.cat((y, x), dim=-1)


class SparseFlashAttentionRope(nn.Module):
    def __init__(
        self,
        dim: int,
        num_heads: int = 16,
        qkv_bias: bool = False,
        proj_bias: bool = True,
        attn_drop: float = 0.0,
        proj_drop: float = 0.0,
        qk_norm: bool = False,
        norm_layer: nn.Module = nn.LayerNorm,
        rope=None,
        block_size: int = 4,
        topk: int = 32,
    ) -> None:
        super().__init__()
        self.num_heads = num_heads
        head_dim = dim // num_heads
        self.scale = head_dim ** -0.5
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(dim, dim, bias=proj_bias)
        self.proj_drop = nn.Dropout(proj_drop)
        self.q_norm = norm_layer(head_dim) if qk_norm else nn.Identity()
        self.k_norm = norm_layer(head_dim) if qk_norm else nn.Identity()
        self.rope = rope
        gate_linear = nn.Linear(dim, num_heads * 2, bias=True)
        nn.init.zeros_(gate_linear.weight)
        gate_linear.bias.data.copy_(torch.tensor([-1.0, 1.0]).repeat(num_heads))
        self.gate = nn.Sequential(gate_linear, nn.Sigmoid())
        self.block_size = block_size
        self.topk = topk
        self.record_idx = False      # debugging aid: keep the last selected-block table in .last_idx
        self.last_idx = None
        self._rows = _TableRows()    # table length when the rotary module is the reference's own
        self.seq_parallel = None     # a seq_parallel.SequenceParallel: x holds this rank's slice of the views

    def _can_fuse_prologue(self, qkv, x, xpos, N, Bs, d) -> bool:
        """Inference (nothing to differentiate), norms that are LayerNorm(d) with affine or Identity, a 2-D
        rotary module (this package's or the reference's pure-PyTorch one) or none, whole blocks, head
        counts the kernel takes."""
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            return False
        norms = (self.q_norm, self.k_norm)
        ident = all(isinstance(m, nn.Identity) for m in norms)
        ln = all(isinstance(m, nn.LayerNorm) and m.elementwise_affine and m.bias is not None and
                 tuple(m.normalized_shape) == (d,) for m in norms)
        if not (ident or (ln and self.q_norm.eps == self.k_norm.eps)):
            return False
        if xpos is not None and not _is_rope2d(self.rope):
            return False
        return d == 64 and N % Bs == 0 and self.num_heads <= 42

    def _forward_fused(self, qkv, gate, xpos, B, N, H, d, Bs) -> Tensor:
        cos = sin = None
        if xpos is not None:
            rows = self.rope._seq_len(xpos) if isinstance(self.rope, RoPE2D) else self._rows(xpos)
            cos, sin = rope_tables(self.rope, d // 2, rows, qkv.device, qkv.dtype)
        qn = kn = None
        if isinstance(self.q_norm, nn.LayerNorm):
            qn = (self.q_norm.weight, self.q_norm.bias, self.q_norm.eps)
            kn = (self.k_norm.weight, self.k_norm.bias, self.k_norm.eps)
        q, k, v, q_c, k_c, v_c = ops.qkv_prologue(qkv.detach(), H, Bs, xpos, cos, sin, qn, kn)
        if self.seq_parallel is not None:
            # this rank's query blocks against the whole sequence: pooled and token-level K/V are exchanged
            y, idx = self.seq_parallel.attention(q, k, v, q_c, k_c, v_c, gate, Bs, self.topk,
                                                 ops.flash_attn_topk_func, ops.sel_attn_merge_chunked)
            if self.record_idx:
                self.last_idx = idx.detach()
            return self.proj_drop(self.proj(y))
        o_c, idx = ops.flash_attn_topk_func(q_c, k_c, v_c, self.topk)
        if self.record_idx:
            self.last_idx = idx.detach()
        y = ops.sel_attn_merge(q, k, v, idx, gate, o_c, Bs)
        return self.proj_drop(self.proj(y))

    def forward(self, x: Tensor, attn_bias=None, xpos: Optional[Tensor] = None) -> Tensor:
        B, N, C = x.shape
        H = self.num_heads
        d = C // H
        Bs = self.block_size ** 2
        qkv = self.qkv(x)
        gate = self.gate(x).view(B, N, H, 2).permute(0, 2, 1, 3)          # [B,H,N,2] view, no copy
        if qkv.dtype != torch.bfloat16:
            raise RuntimeError("SparseFlashAttentionRope runs in bf16 (use torch.autocast(dtype=torch.bfloat16)); "
                               f"got {qkv.dtype}")
        gate = gate.to(qkv.dtype)
        if self._can_fuse_prologue(qkv, x, xpos, N, Bs, d):
            return self._forward_fused(qkv, gate, xpos, B, N, H, d, Bs)
        if self.seq_parallel is not None and N % Bs != 0:
            raise RuntimeError("sequence-parallel attention needs whole 16-token blocks on every rank")
        qkv5 = qkv.view(B, N, 3, H, d)
        q_t, k_t, v_t = (qkv5[:, :, i].permute(0, 2, 1, 3) for i in range(3))   # [B,H,N,d] views of the projection

        # compression branch: pool raw q,k,v, then norm + rope with the block's mean position
        q_c, k_c, v_c = (ops.pool_tokens(t, Bs, Bs) for t in (q_t, k_t, v_t))
        q_c, k_c = self.q_norm(q_c).to(v_c.dtype), self.k_norm(k_c).to(v_c.dtype)
        rope_kw = {}
        if xpos is not None and isinstance(self.rope, RoPE2D):
            rope_kw = dict(seq_len=self.rope._seq_len(xpos))     # one table for token and block positions
        if xpos is not None:
            xpos_c = xpos.view(B, N // Bs, Bs, 2).float().mean(dim=2).int()
            q_c = self.rope(q_c, xpos_c, **rope_kw)
            k_c = self.rope(k_c, xpos_c, **rope_kw)
        # selection branch at token level, gated merge fused into its epilogue
        q, k = self.q_norm(q_t).to(qkv.dtype), self.k_norm(k_t).to(qkv.dtype)
        if xpos is not None:
            q = self.rope(q, xpos, **rope_kw)
            k = self.rope(k, xpos, **rope_kw)
        if self.seq_parallel is not None:
            # this rank's queries against the whole sequence; the backward reduce-scatters dK and dV
            y, idx = self.seq_parallel.attention_grad(q.contiguous(), k.contiguous(), v_t.contiguous(), q_c, k_c, v_c,
                                                      gate, Bs, self.topk, ops.flash_attn_topk_func, ops.sel_attn_merge)
        else:
            o_c, idx = ops.flash_attn_topk_func(q_c, k_c, v_c, self.topk)
            y = ops.sel_attn_merge(q.contiguous(), k.contiguous(), v_t.contiguous(), idx, gate, o_c, Bs)
        if self.record_idx:
            self.last_idx = idx.detach()
        y = self.proj(y)
        return self.proj_drop(y)
