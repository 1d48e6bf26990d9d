"""The sparse global-attention op for callers whose q, k, v live in pinned HOST memory.

The reference keeps its tensors on the device (`SparseFlashAttentionRope.forward`,
pi3/models/layers/sparse_attention.py:88-143); a host that holds them in its own memory pays the
PCIe copies on top of the kernels.  `HostPipeline` hides most of that cost by cutting the op along
the two axes on which it is independent and running three streams:

* copy-in stream: K and V arrive head group by head group (a head of a `[1,H,T,d]` tensor is one
  contiguous span) and are pooled as they land; the queries follow in chunks of query blocks;
* compute stream: per query chunk, pool -> compression attention + top-k -> selection attention
  with the gated merge; a chunk needs all pooled K/V but only its own queries;
* copy-out stream: each chunk of `y [1,T,H*d]` (token-major, so a chunk is contiguous) goes back
  while the next chunk computes.

The query chunk is sized so that one compression-attention launch fills whole waves of the GPU
(`H * ceil(rows/256)` CTAs a multiple of the SM count).  Results are bit-identical to the unchunked
call: every query row sees the same keys in the same order.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from . import ops

_ROWS_PER_CTA = 256          # pooled query rows one compression-attention CTA owns


def rows_per_chunk_for(num_heads: int, sm_count: int) -> int:
    """Pooled query rows per chunk such that one compression-attention launch (``num_heads *
    ceil(rows/256)`` CTAs, one CTA per SM at a time) fills whole waves of the GPU."""
    return _ROWS_PER_CTA * (sm_count // math.gcd(num_heads, sm_count))


def query_chunks(num_pooled_rows: int, rows_per_chunk: int):
    """[(first pooled row, last pooled row + 1)] covering ``num_pooled_rows`` in order; the last may be short."""
    rows = max(1, min(num_pooled_rows, rows_per_chunk))
    return [(r, min(num_pooled_rows, r + rows)) for r in range(0, num_pooled_rows, rows)]


def _pinned(t: Tensor, name: str) -> None:
    if t.device.type != "cpu" or not t.is_pinned():
        raise RuntimeError(f"{name}: expected a pinned host tensor")
    if t.dtype != torch.bfloat16 or not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous bf16 tensor")


class HostPipeline:
    """Pre-allocated device buffers and streams for one problem size (B = 1).

    ``pipe = HostPipeline(H, T, device=...)`` then ``pipe(hq, hk, hv, hgate, hy)`` with pinned host
    tensors ``hq/hk/hv [1,H,T,d]``, ``hgate [1,H,T,2]`` and the result buffer ``hy [1,T,H*d]``.
    The call only enqueues work; the calling stream is made to wait for the last copy, so an event
    recorded on it (or a synchronize) covers the whole op."""

    def __init__(self, H: int, T: int, d: int = 64, block_size: int = 16, topk: int = 32,
                 device: Optional[torch.device] = None, rows_per_chunk: Optional[int] = None,
                 heads_per_copy: int = 2):
        if T % block_size:
            raise RuntimeError(f"T={T} must be a multiple of the block size {block_size}")
        self.H, self.T, self.d, self.block, self.topk = H, T, d, block_size, topk
        self.dev = torch.device(device if device is not None else torch.cuda.current_device())
        if self.dev.type != "cuda":
            raise RuntimeError("HostPipeline needs a CUDA device")
        self.Nc = T // block_size
        if rows_per_chunk is None:
            sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
            rows_per_chunk = rows_per_chunk_for(H, sms)
        self.rows = max(1, min(self.Nc, rows_per_chunk))
        self.heads_per_copy = max(1, min(H, heads_per_copy))
        bf = dict(device=self.dev, dtype=torch.bfloat16)
        self.k = torch.empty(1, H, T, d, **bf)
        self.v = torch.empty(1, H, T, d, **bf)
        self.k_c = torch.empty(1, H, self.Nc, d, **bf)
        self.v_c = torch.empty(1, H, self.Nc, d, **bf)
        self.gate = torch.empty(1, H, T, 2, **bf)
        tc = self.rows * block_size
        self.qbuf = [torch.empty(1, H, tc, d, **bf) for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)

    def chunks(self):
        """[(first pooled row, last pooled row + 1)] of the query chunks."""
        return query_chunks(self.Nc, self.rows)

    @torch.no_grad()
    def __call__(self, hq: Tensor, hk: Tensor, hv: Tensor, hgate: Tensor, hy: Tensor) -> None:
        H, T, d, bs = self.H, self.T, self.d, self.block
        for n, t, shape in (("hq", hq, (1, H, T, d)), ("hk", hk, (1, H, T, d)), ("hv", hv, (1, H, T, d)),
                            ("hgate", hgate, (1, H, T, 2)), ("hy", hy, (1, T, H * d))):
            _pinned(t, n)
            if tuple(t.shape) != shape:
                raise RuntimeError(f"{n}: expected shape {shape}, got {tuple(t.shape)}")
        main = torch.cuda.current_stream(self.dev)
        s_in, s_out = self.s_in, self.s_out
        s_in.wait_stream(main)            # device buffers may still be read by an earlier call
        s_out.wait_stream(main)

        # K and V, head group by head group; each group is pooled on the compute stream as it lands
        hp = self.heads_per_copy
        for src, dst, dst_c in ((hk, self.k, self.k_c), (hv, self.v, self.v_c)):
            for h0 in range(0, H, hp):
                h1 = min(H, h0 + hp)
                with torch.cuda.stream(s_in):
                    dst[:, h0:h1].copy_(src[:, h0:h1], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(s_in)
                main.wait_event(landed)
                dst_c[:, h0:h1].copy_(ops.pool_tokens(dst[:, h0:h1], bs, bs))
        with torch.cuda.stream(s_in):
            self.gate.copy_(hgate, non_blocking=True)

        # queries in chunks: copy-in (per head, contiguous spans) | compute | copy-out
        q_free = [None, None]             # compute of the chunk that last used qbuf[i] is finished
        for c, (r0, r1) in enumerate(self.chunks()):
            i = c & 1
            t0, t1 = r0 * bs, r1 * bs
            q_dev = self.qbuf[i].view(-1)[:H * (t1 - t0) * d].view(1, H, t1 - t0, d)
            with torch.cuda.stream(s_in):
                if q_free[i] is not None:
                    s_in.wait_event(q_free[i])
                for h in range(H):
                    q_dev[0, h].copy_(hq[0, h, t0:t1], non_blocking=True)
                landed = torch.cuda.Event()
                landed.record(s_in)
            main.wait_event(landed)
            q_c = ops.pool_tokens(q_dev, bs, bs)
            o_c, idx = ops.flash_attn_topk_func(q_c, self.k_c, self.v_c, self.topk)
            y = ops.sel_attn_merge(q_dev, self.k, self.v, idx, self.gate[:, :, t0:t1], o_c, bs)
            done = torch.cuda.Event()
            done.record(main)
            q_free[i] = done
            y.record_stream(s_out)        # the allocator must not hand y out again before it has left
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                hy[:, t0:t1].copy_(y, non_blocking=True)
        main.wait_stream(s_out)
        main.wait_stream(s_in)
