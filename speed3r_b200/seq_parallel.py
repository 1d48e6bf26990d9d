"""Sequence-partitioned sparse global attention (one process per GPU).

The reference is single-GPU (it scales to long sequences by sparsity only); this is the
multi-GPU form of its op.  Token order is view-major (pi3/models/pi3_sparse.py:250-251), so a
contiguous partition of query blocks is a contiguous partition of views:

* rank r owns tokens ``[r*T/G, (r+1)*T/G)`` and every query block inside them;
* the pooled keys/values are all-gathered (one exchange, 2*Nc*H*d*2 bytes in total);
* the token-level keys/values are all-gathered into the chunked layout
  ``[G, B, H, T/G, d]`` that the selection kernel reads in place (its K/V gathers then hit local
  HBM only);
* everything else (pooling, compression attention of the local query rows against all pooled
  keys, selection attention of the local query blocks, gated merge) is local.

The two attention callables are injected so that the host logic can be exercised on CPU ranks
(gloo) with the oracle standing in for the kernels.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def partition(T: int, block: int, world: int, rank: int) -> Tuple[int, int]:
    """Token range ``[t0, t1)`` of ``rank``: whole query blocks, sizes equal (T must split evenly)."""
    if T % (block * world) != 0:
        raise ValueError(f"T={T} must be a multiple of block*world = {block * world}")
    per = T // world
    return rank * per, (rank + 1) * per


def all_gather_chunks(x: Tensor, group=None) -> Tensor:
    """``x [B,H,n,d]`` on every rank -> ``[G,B,H,n,d]`` (chunk g = rank g's tensor)."""
    world = dist.get_world_size(group)
    # the output is laid out as the ranks' tensors concatenated along dim 0 (both NCCL and gloo
    # accept this form); viewed as [G, ...] afterwards
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out.view((world,) + tuple(x.shape))


def chunks_to_dense(xc: Tensor) -> Tensor:
    """``[G,B,H,n,d]`` -> ``[B,H,G*n,d]`` (sequence order restored)."""
    G, B, H, n, d = xc.shape
    return xc.permute(1, 2, 0, 3, 4).reshape(B, H, G * n, d)


def sparse_attention_partitioned(q: Tensor, k: Tensor, v: Tensor, gate: Tensor, block: int, topk: int,
                                 pool: Callable, cmp_attn_topk: Callable, sel_attn_merge: Callable,
                                 group=None, side_stream: Optional["torch.cuda.Stream"] = None, side_group=None):
    """Local shard of the op.  ``q,k,v [B,H,T/G,d]`` and ``gate [B,H,T/G,2]`` are this rank's tokens.

    ``pool(x, kernel, stride)``; ``cmp_attn_topk(q_c, k_c, v_c, topk) -> (o_c, idx)``;
    ``sel_attn_merge(q, k_chunks, v_chunks, idx, gate, o_c, block) -> y [B,T/G,H*d]`` with K/V in
    the chunked ``[G,B,H,T/G,d]`` layout.  Returns ``(y_local, idx_local)``.

    With ``side_stream`` the token-level all-gather (the large one) runs on that stream while
    the compression attention, which only needs pooled data, runs on the current stream.  With a
    ``side_group`` as well (a second process group over the same ranks, i.e. its own communicator)
    the large all-gather is issued first and the pooled ones run beside it instead of ahead of it.
    """
    k_all = v_all = None
    cur = torch.cuda.current_stream() if side_stream is not None else None
    if side_stream is not None and side_group is not None:
        side_stream.wait_stream(cur)              # k and v are ready on the current stream
        with torch.cuda.stream(side_stream):
            k_all, v_all = all_gather_chunks(k, side_group), all_gather_chunks(v, side_group)
    q_c, k_c, v_c = pool(q, block, block), pool(k, block, block), pool(v, block, block)
    kc_all = chunks_to_dense(all_gather_chunks(k_c, group))
    vc_all = chunks_to_dense(all_gather_chunks(v_c, group))
    if side_stream is not None:
        if k_all is None:
            side_stream.wait_stream(cur)
            with torch.cuda.stream(side_stream):
                k_all, v_all = all_gather_chunks(k, group), all_gather_chunks(v, group)
        o_c, idx = cmp_attn_topk(q_c, kc_all, vc_all, topk)
        cur.wait_stream(side_stream)
        k_all.record_stream(cur)
        v_all.record_stream(cur)
    else:
        k_all, v_all = all_gather_chunks(k, group), all_gather_chunks(v, group)
        o_c, idx = cmp_attn_topk(q_c, kc_all, vc_all, topk)
    y = sel_attn_merge(q, k_all, v_all, idx, gate, o_c, block)
    return y, idx
