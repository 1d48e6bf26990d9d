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

The token-level exchange is the large one (2*T*H*d*2 bytes in total) and is only needed by the
selection kernel, i.e. after the compression attention.  An NCCL all-gather moves it with CTAs that
compete with the compression kernel for SMs; ``PeerGather`` pulls it instead with a copy kernel of a
few CTAs from buffers every rank exposes through CUDA IPC, launched just ahead of the compression
kernel, which then has all the other SMs to itself from the start.
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


_IPC_BASE = {}      # (importing device, IPC handle) -> base address of the mapped allocation in this process


class PeerGather:
    """All-gather of equally shaped ``[B,H,n,d]`` shards by peer loads (one node, one process per GPU).

    Every rank owns the result buffer ``out [G,B,H,n,d]`` (chunk g = rank g's shard, the layout the
    selection kernel reads in place) and has mapped its peers' result buffers through CUDA IPC; a rank
    writes its own shard into ``out[rank]`` and pulls shard g from rank g's ``out[g]``.

    Protocol of one exchange, all calls on the caller's current stream unless said otherwise:

    1. ``stage(x)`` - wait until every rank has finished pulling the previous exchange (a one-element
       all-reduce: a rank reaches it only after its own pulls), then copy the local shard into
       ``out[rank]`` (a producer may instead write ``local()`` directly and call ``stage(None)``);
    2. some collective of the caller that every rank enters AFTER ``stage`` (here: the pooled all-gather)
       - once it has completed locally, every peer's shard is known to be written;
    3. ``pull()`` - a side stream waits for the current stream (or for a given event), then a copy kernel
       of a few CTAs (``s3r_peer_pull``: plain loads from the peers, stores locally) fills ``out``;
    4. ``wait()`` - the current stream waits for the side streams; ``out`` is complete.

    Peers' memory is only ever the SOURCE of plain copies."""

    def __init__(self, shape, dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.shape = tuple(shape)
        self.out = torch.empty((self.world,) + self.shape, device=device, dtype=dtype)
        self._token = torch.zeros(1, device=device)
        # Every rank exports its buffer (handle of the allocation + offset) and imports its peers' with its
        # own device current: the addresses are then valid for kernels of THIS device.
        import ctypes as C
        from . import _lib
        lib = _lib.load()
        with torch.cuda.device(device):
            hbuf = C.create_string_buffer(64)
            off = C.c_int64(0)
            _lib.check(lib.s3r_ipc_export(self.out.data_ptr(), hbuf, C.byref(off)), "s3r_ipc_export")
            mine = (hbuf.raw, int(off.value))
            exported = [None] * self.world
            dist.all_gather_object(exported, mine, group=group)
            shard_bytes = self.out[0].numel() * self.out.element_size()
            self.peer_ptr = []                       # device address of rank g's own shard inside rank g's buffer
            for g, (handle, offset) in enumerate(exported):
                if g == self.rank:
                    self.peer_ptr.append(self.out[g].data_ptr())
                    continue
                key = (torch.device(device).index, handle)
                if key not in _IPC_BASE:             # an allocation is opened once per process and device
                    ptr = C.c_void_p(0)
                    _lib.check(lib.s3r_ipc_import(handle, 0, C.byref(ptr)), "s3r_ipc_import")
                    _IPC_BASE[key] = int(ptr.value)
                self.peer_ptr.append(_IPC_BASE[key] + offset + g * shard_bytes)
        self.streams = [torch.cuda.Stream(device=device, priority=-1)]
        self._done = [torch.cuda.Event() for _ in self.streams]
        dist.barrier(group=group)                    # every rank has mapped every buffer before first use

    def local(self) -> Tensor:
        """This rank's slot of the result buffer, ``[B,H,n,d]``."""
        return self.out[self.rank]

    def stage(self, x: Optional[Tensor]) -> None:
        dist.all_reduce(self._token, group=self.group)       # nobody is still reading the previous contents
        if x is not None:
            self.out[self.rank].copy_(x)

    def pull(self, after: Optional["torch.cuda.Event"] = None, ctas: int = 16) -> Tensor:
        """Launch the copy kernel on the side stream; it starts once the current stream has reached this
        point or, with ``after``, once that event has happened.  Call it BEFORE launching the kernel it is to
        run beside: its few CTAs must be resident first."""
        import ctypes as C
        from . import _lib
        cur = torch.cuda.current_stream()
        st = self.streams[0]
        if after is not None:
            st.wait_event(after)
        else:
            st.wait_stream(cur)
        n = self.world - 1
        srcs = (C.c_void_p * n)()
        dsts = (C.c_void_p * n)()
        nbytes = (C.c_int64 * n)()
        for i in range(1, self.world):                        # the ring after this rank
            g = (self.rank + i) % self.world
            srcs[i - 1] = self.peer_ptr[g]
            dsts[i - 1] = self.out[g].data_ptr()
            nbytes[i - 1] = self.out[g].numel() * self.out.element_size()
        with torch.cuda.device(self.out.device):
            _lib.check(_lib.load().s3r_peer_pull(srcs, dsts, nbytes, n, ctas, st.cuda_stream), "s3r_peer_pull")
        self._done[0].record(st)
        return self.out

    def wait(self) -> Tensor:
        cur = torch.cuda.current_stream()
        for ev in self._done:
            cur.wait_event(ev)
        return self.out


def chunks_to_dense(xc: Tensor) -> Tensor:
    """``[G,B,H,n,d]`` -> ``[B,H,G*n,d]`` (sequence order restored)."""
    G, B, H, n, d = xc.shape
    return xc.permute(1, 2, 0, 3, 4).reshape(B, H, G * n, d)


def all_gather_pooled(k_c: Tensor, v_c: Tensor, group=None) -> Tuple[Tensor, Tensor]:
    """Pooled keys and values of all ranks as dense ``[B,H,Nc,d]`` tensors, through ONE all-gather (the
    compression kernel waits for both, and at eight ranks a second collective launch is a visible share of
    the step)."""
    g = all_gather_chunks(torch.stack((k_c, v_c)), group)            # [G,2,B,H,n,d]
    return chunks_to_dense(g[:, 0]), chunks_to_dense(g[:, 1])


def sparse_attention_partitioned(q: Tensor, k: Tensor, v: Tensor, gate: Tensor, block: int, topk: int,
                                 pool: Callable, cmp_attn_topk: Callable, sel_attn_merge: Callable,
                                 group=None, side_stream: Optional["torch.cuda.Stream"] = None, side_group=None,
                                 peer_gather: Optional[Tuple["PeerGather", "PeerGather"]] = None,
                                 pooled: Optional[Tuple[Tensor, Tensor, Tensor]] = None):
    """Local shard of the op.  ``q,k,v [B,H,T/G,d]`` and ``gate [B,H,T/G,2]`` are this rank's tokens.

    ``pool(x, kernel, stride)``; ``cmp_attn_topk(q_c, k_c, v_c, topk) -> (o_c, idx)``;
    ``sel_attn_merge(q, k_chunks, v_chunks, idx, gate, o_c, block) -> y [B,T/G,H*d]`` with K/V in
    the chunked ``[G,B,H,T/G,d]`` layout.  Returns ``(y_local, idx_local)``.

    With ``side_stream`` the token-level all-gather (the large one) runs on that stream while
    the compression attention, which only needs pooled data, runs on the current stream.  With a
    ``side_group`` as well (a second process group over the same ranks, i.e. its own communicator)
    the large all-gather is issued first and the pooled ones run beside it instead of ahead of it.
    With ``peer_gather = (PeerGather for k, PeerGather for v)`` the token-level exchange runs on the copy
    engines instead (see ``PeerGather``); the pooled all-gather is the collective that orders it.
    ``pooled = (q_c, k_c, v_c)`` of the local tokens skips the pooling (a caller whose prologue has
    produced them already, with its own normalisation and rotary embedding).
    """
    def pooled_local():
        if pooled is not None:
            return pooled
        return pool(q, block, block), pool(k, block, block), pool(v, block, block)

    if peer_gather is not None:
        pk, pv = peer_gather
        pk.stage(k)
        pv.stage(v)
        q_c, k_c, v_c = pooled_local()
        kc_all, vc_all = all_gather_pooled(k_c, v_c, group)
        pk.pull()                                              # few CTAs, resident before the attention kernel
        pv.pull()
        o_c, idx = cmp_attn_topk(q_c, kc_all, vc_all, topk)
        k_all, v_all = pk.wait(), pv.wait()
        y = sel_attn_merge(q, k_all, v_all, idx, gate, o_c, block)
        return y, idx
    k_all = v_all = None
    cur = torch.cuda.current_stream() if side_stream is not None else None
    if side_stream is not None and side_group is not None:
        side_stream.wait_stream(cur)              # k and v are ready on the current stream
        with torch.cuda.stream(side_stream):
            k_all, v_all = all_gather_chunks(k, side_group), all_gather_chunks(v, side_group)
    q_c, k_c, v_c = pooled_local()
    kc_all, vc_all = all_gather_pooled(k_c, v_c, group)
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


class _GatherSeq(torch.autograd.Function):
    """All-gather of ``x [B,H,n,d]`` along the sequence into ``[B,H,G*n,d]`` (rank order = sequence order).
    Its backward is the matching reduce-scatter: every rank holds gradient contributions to ALL tokens (from
    its own queries) and receives the sum over ranks of the contributions to its own tokens."""

    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        return chunks_to_dense(all_gather_chunks(x.contiguous(), group))

    @staticmethod
    def backward(ctx, g: Tensor):
        world = dist.get_world_size(ctx.group)
        B, H, T, d = g.shape
        n = T // world
        chunks = g.reshape(B, H, world, n, d).permute(2, 0, 1, 3, 4).contiguous()      # [G,B,H,n,d]
        if dist.get_backend(ctx.group) == "gloo":            # no reduce-scatter there: reduce, keep the own chunk
            dist.all_reduce(chunks, group=ctx.group)
            return chunks[dist.get_rank(ctx.group)].clone(), None
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter_tensor(out, chunks, group=ctx.group)
        return out, None


def sparse_attention_partitioned_grad(q: Tensor, k: Tensor, v: Tensor, gate: Tensor, block: int, topk: int,
                                      pool: Callable, cmp_attn_topk: Callable, sel_attn_merge: Callable,
                                      group=None, pooled: Optional[Tuple[Tensor, Tensor, Tensor]] = None):
    """The differentiable form of ``sparse_attention_partitioned`` (training on sequences longer than one
    GPU holds): same arguments, but ``cmp_attn_topk`` and ``sel_attn_merge`` are the differentiable ops and
    take K/V as dense ``[B,H,T,d]`` tensors.  Gradients with respect to this rank's ``q`` and ``gate`` are
    local; those with respect to ``k``, ``v`` (and the pooled ``k_c``, ``v_c``) are computed by every rank for
    all keys from its own queries and reduce-scattered by the backward of the all-gathers.  The partial
    gradients are rounded to the tensors' dtype before the reduction, so the result differs from the
    single-GPU gradient by that rounding (it is not bit-equal as the forward is)."""
    if pooled is None:
        pooled = (pool(q, block, block), pool(k, block, block), pool(v, block, block))
    q_c, k_c, v_c = pooled
    kc_all, vc_all = _GatherSeq.apply(k_c, group), _GatherSeq.apply(v_c, group)
    k_all, v_all = _GatherSeq.apply(k, group), _GatherSeq.apply(v, group)
    o_c, idx = cmp_attn_topk(q_c, kc_all, vc_all, topk)
    y = sel_attn_merge(q, k_all, v_all, idx, gate, o_c, block)
    return y, idx


class SequenceParallel:
    """What the drop-in module needs to run its two attention branches sequence-partitioned: set
    ``module.seq_parallel = SequenceParallel(group)`` on every global-attention module of a model whose
    ranks each hold a contiguous slice of the views (token order is view-major).  The module's own
    prologue (split, LayerNorm, rotary embedding, pooling) stays local; this object does the exchange:
    ``attention`` for inference (chunked K/V, exchange overlapped with the compression kernel),
    ``attention_grad`` when gradients are needed (dense K/V, reduce-scatter of dK/dV in the backward)."""

    def __init__(self, group=None, gather: str = "nccl"):
        self.group = group
        self.gather = gather
        self._peer = {}
        self._side = None
        self._side_group = None

    def attention(self, q: Tensor, k: Tensor, v: Tensor, q_c: Tensor, k_c: Tensor, v_c: Tensor, gate: Tensor,
                  block: int, topk: int, cmp_attn_topk: Callable, sel_attn_merge: Callable):
        kw = {}
        if self.gather == "peer":
            key = (tuple(k.shape), k.dtype, k.device)
            if key not in self._peer:
                self._peer[key] = (PeerGather(k.shape, k.dtype, k.device, self.group),
                                   PeerGather(k.shape, k.dtype, k.device, self.group))
            kw["peer_gather"] = self._peer[key]
        else:
            if self._side is None:
                self._side = torch.cuda.Stream(priority=-1)
                self._side_group = dist.new_group(list(range(dist.get_world_size(self.group))))
            kw.update(side_stream=self._side, side_group=self._side_group)
        return sparse_attention_partitioned(q, k, v, gate, block, topk, None, cmp_attn_topk, sel_attn_merge,
                                            group=self.group, pooled=(q_c, k_c, v_c), **kw)

    def attention_grad(self, q: Tensor, k: Tensor, v: Tensor, q_c: Tensor, k_c: Tensor, v_c: Tensor, gate: Tensor,
                       block: int, topk: int, cmp_attn_topk: Callable, sel_attn_merge: Callable):
        return sparse_attention_partitioned_grad(q, k, v, gate, block, topk, None, cmp_attn_topk, sel_attn_merge,
                                                 group=self.group, pooled=(q_c, k_c, v_c))
