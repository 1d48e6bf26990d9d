"""The sparse global-attention op for callers whose q, k, v live in pinned HOST memory.

The reference keeps its tensors on the device (`SparseFlashAttentionRope.forward`,
pi3/models/layers/sparse_attention.py:88-143); a host that holds them in its own memory pays the
PCIe copies on top of the kernels.  `HostPipeline` hides most of that cost by cutting the op along
the two axes on which it is independent and running three streams:

* heads are independent, so the op runs head group by head group: a group's K and V arrive (a head of a
  `[1,H,T,d]` tensor is one contiguous span) and are pooled as they land, then its queries follow in
  chunks of query blocks.  The first group computes while the second is still on the bus, so the copy-in
  stream never waits for the kernels and the kernels only wait for data;
* compute stream: per (head group, query chunk), pool -> compression attention + top-k -> selection
  attention with the gated merge; a chunk needs the group's pooled K/V but only its own queries;
* copy-out stream: each chunk of a group's `y [1,T,Hg*d]` goes back while the next chunk computes, as a
  strided copy into the group's columns of the caller's `y [1,T,H*d]`.

The query chunk is sized so that one compression-attention launch fills whole waves of the GPU
(`Hg * ceil(rows/256)` CTAs a multiple of the SM count).  Results are bit-identical to the unchunked
call: every query row sees the same keys in the same order.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor

from . import _lib, ops

_ROWS_PER_CTA = 256          # pooled query rows one compression-attention CTA owns
_Q_BUFFERS = 4


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
    recorded on it (or a synchronize) covers the whole op.  ``heads_per_group`` heads travel and compute
    together (``heads_per_copy`` is the older name of the same argument)."""

    def __init__(self, H: int, T: int, d: int = 64, block_size: int = 16, topk: int = 32,
                 device: Optional[torch.device] = None, rows_per_chunk: Optional[int] = None,
                 heads_per_group: Optional[int] = None, heads_per_copy: Optional[int] = None):
        if T % block_size:
            raise RuntimeError(f"T={T} must be a multiple of the block size {block_size}")
        self.H, self.T, self.d, self.block, self.topk = H, T, d, block_size, topk
        self.dev = torch.device(device if device is not None else torch.cuda.current_device())
        if self.dev.type != "cuda":
            raise RuntimeError("HostPipeline needs a CUDA device")
        self.Nc = T // block_size
        hg = heads_per_group if heads_per_group is not None else heads_per_copy
        self.hg = max(1, min(H, hg if hg is not None else 4))
        if rows_per_chunk is None:
            sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
            rows_per_chunk = rows_per_chunk_for(self.hg, sms)
        self.rows = max(1, min(self.Nc, rows_per_chunk))
        bf = dict(device=self.dev, dtype=torch.bfloat16)
        hg = self.hg
        # two sets of group buffers: group g+1 lands while group g computes
        self.k = [torch.empty(1, hg, T, d, **bf) for _ in range(2)]
        self.v = [torch.empty(1, hg, T, d, **bf) for _ in range(2)]
        self.gate = [torch.empty(1, hg, T, 2, **bf) for _ in range(2)]
        tc = self.rows * block_size
        # query chunks may run up to four ahead of the kernels: a chunk computes a little longer than it travels, and
        # the copy-in stream must not wait for a free buffer while the next group's K and V could be on the bus
        self.qbuf = [torch.empty(1, hg, tc, d, **bf) for _ in range(_Q_BUFFERS)]
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)

    def chunks(self):
        """[(first pooled row, last pooled row + 1)] of the query chunks (the same for every head group)."""
        return query_chunks(self.Nc, self.rows)

    def groups(self):
        """[(first head, last head + 1)] of the head groups; the last may be short."""
        return [(h, min(self.H, h + self.hg)) for h in range(0, self.H, self.hg)]

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
        lib = _lib.load()
        esz = hy.element_size()

        grp_free = [None, None]           # compute of the group that last used buffer set i is finished
        q_free = [None] * _Q_BUFFERS      # compute of the chunk that last used qbuf[i] is finished
        step = 0
        for gi, (h0, h1) in enumerate(self.groups()):
            b, n = gi & 1, h1 - h0
            k, v, gate = (buf[b][:, :n] for buf in (self.k, self.v, self.gate))
            with torch.cuda.stream(s_in):
                if grp_free[b] is not None:
                    s_in.wait_event(grp_free[b])
                k.copy_(hk[:, h0:h1], non_blocking=True)
                k_in = torch.cuda.Event()
                k_in.record(s_in)
                v.copy_(hv[:, h0:h1], non_blocking=True)
                gate.copy_(hgate[:, h0:h1], non_blocking=True)
                v_in = torch.cuda.Event()
                v_in.record(s_in)
            main.wait_event(k_in)
            k_c = ops.pool_tokens(k, bs, bs)                      # pooled while V is still on the bus
            main.wait_event(v_in)
            v_c = ops.pool_tokens(v, bs, bs)
            done = None
            for r0, r1 in self.chunks():
                i = step % _Q_BUFFERS
                step += 1
                t0, t1 = r0 * bs, r1 * bs
                q_dev = self.qbuf[i].view(-1)[:n * (t1 - t0) * d].view(1, n, t1 - t0, d)
                with torch.cuda.stream(s_in):
                    if q_free[i] is not None:
                        s_in.wait_event(q_free[i])
                    for h in range(n):                            # per head: contiguous spans on both sides
                        q_dev[0, h].copy_(hq[0, h0 + h, t0:t1], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(s_in)
                main.wait_event(landed)
                q_c = ops.pool_tokens(q_dev, bs, bs)
                o_c, idx = ops.flash_attn_topk_func(q_c, k_c, v_c, self.topk)
                y = ops.sel_attn_merge(q_dev, k, v, idx, gate[:, :, t0:t1], o_c, bs)      # [1, t1-t0, n*d]
                done = torch.cuda.Event()
                done.record(main)
                q_free[i] = done
                y.record_stream(s_out)    # the allocator must not hand y out again before it has left
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    # this group's columns of the rows t0..t1 of hy [1,T,H*d]
                    _lib.check(lib.s3r_copy2d_async(hy.data_ptr() + (t0 * H * d + h0 * d) * esz, H * d * esz,
                                                    y.data_ptr(), n * d * esz, n * d * esz, t1 - t0,
                                                    s_out.cuda_stream), "s3r_copy2d_async")
            grp_free[b] = done
        main.wait_stream(s_out)
        main.wait_stream(s_in)
