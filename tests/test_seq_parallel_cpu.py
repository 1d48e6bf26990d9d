"""Host logic of the sequence-partitioned op on CPU ranks (gloo, world_size 2), with the oracle
standing in for the kernels: the shards put together must equal the single-process result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import restatement as R
from speed3r_b200 import seq_parallel

B, H, T, D, BS, K = 1, 2, 512, 64, 16, 8


def _inputs():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(B, H, T, D, generator=g) for _ in range(3))
    gate = torch.sigmoid(torch.randn(B, H, T, 2, generator=g))
    return q, k, v, gate


def _sel_chunked(q, k_chunks, v_chunks, idx, gate, o_c, block):
    k = seq_parallel.chunks_to_dense(k_chunks)
    v = seq_parallel.chunks_to_dense(v_chunks)
    o_s, _ = R.sel_attn(q, k, v, idx, block)
    return R.gated_merge(gate, o_c, o_s, block)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, gate = _inputs()
        t0, t1 = seq_parallel.partition(T, BS, world, rank)
        sl = slice(t0, t1)
        y, idx = seq_parallel.sparse_attention_partitioned(
            q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(), gate[:, :, sl].contiguous(),
            BS, K, R.pool_tokens, lambda a, b, c, kk: (lambda o: (o[0], o[2]))(R.cmp_attn_topk(a, b, c, kk)),
            _sel_chunked)
        torch.save((y, idx), os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_partition_is_even_and_block_aligned():
    assert seq_parallel.partition(1008 * 8, 16, 4, 1) == (2016, 4032)
    with pytest.raises(ValueError):
        seq_parallel.partition(1000, 16, 3, 0)


def test_chunks_to_dense_restores_sequence_order():
    x = torch.arange(2 * 1 * 2 * 3 * 4).float().view(2, 1, 2, 3, 4)     # [G,B,H,n,d]
    d = seq_parallel.chunks_to_dense(x)
    assert d.shape == (1, 2, 6, 4)
    assert torch.equal(d[0, 1, 3:], x[1, 0, 1])


def test_two_ranks_match_single_process(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    q, k, v, gate = _inputs()
    y_ref, idx_ref = R.sparse_attention_op(q, k, v, gate, BS, K, BS, BS)
    ys, idxs = zip(*(torch.load(os.path.join(tmp_path, f"r{r}.pt")) for r in range(2)))
    assert torch.equal(torch.cat(idxs, dim=2), idx_ref)
    torch.testing.assert_close(torch.cat(ys, dim=1), y_ref, atol=1e-5, rtol=1e-5)


def _worker_grad(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, gate = _inputs()
        t0, t1 = seq_parallel.partition(T, BS, world, rank)
        ql, kl, vl, gl = (t[:, :, t0:t1].clone().requires_grad_(True) for t in (q, k, v, gate))
        y, idx = seq_parallel.sparse_attention_partitioned_grad(
            ql, kl, vl, gl, BS, K, R.pool_tokens, lambda a, b, c, kk: (lambda o: (o[0], o[2]))(R.cmp_attn_topk(a, b, c, kk)),
            lambda qq, kk, vv, ii, gg, oc, bs: R.gated_merge(gg, oc, R.sel_attn(qq, kk, vv, ii, bs)[0], bs))
        dy = torch.randn(B, T, H * D, generator=torch.Generator().manual_seed(5))[:, t0:t1]
        y.backward(dy)
        torch.save((y.detach(), ql.grad, kl.grad, vl.grad, gl.grad), os.path.join(out_dir, f"g{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gradients_match_single_process(tmp_path):
    """dQ and dgate are local; dK and dV of a rank's tokens are the sum over ranks of the contributions of
    their queries (the backward of the all-gather is a reduce-scatter)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_grad, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    q, k, v, gate = (t.clone().requires_grad_(True) for t in _inputs())
    y_ref, _ = R.sparse_attention_op(q, k, v, gate, BS, K, BS, BS)
    dy = torch.randn(B, T, H * D, generator=torch.Generator().manual_seed(5))
    y_ref.backward(dy)
    parts = [torch.load(os.path.join(tmp_path, f"g{r}.pt")) for r in range(2)]
    torch.testing.assert_close(torch.cat([p[0] for p in parts], dim=1), y_ref.detach(), atol=1e-5, rtol=1e-5)
    for i, ref in ((1, q.grad), (2, k.grad), (3, v.grad), (4, gate.grad)):
        torch.testing.assert_close(torch.cat([p[i] for p in parts], dim=2), ref, atol=2e-5, rtol=1e-4)
