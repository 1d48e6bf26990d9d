"""The drop-in at the sizes and inside the callers the reference uses it in.

* the module at the reference's training size (B=2, 24 views of 224x224 -> T = 6144 tokens per sample,
  1024 channels, 16 heads), forward and backward, against the CPU oracle;
* the module inside the reference's own ``BlockRope`` and ``Pi3_Sparse`` (unmodified reference code from
  ``baseline/_ref``, filled by ``baseline/install_ref.sh``; skipped when that folder is absent): the
  reference's Triton attention class and this package's class, same weights, same inputs;
* the sequence-partitioned op on 2+ GPUs against the single-GPU op (skipped below 2 GPUs).
"""
import os
import sys

import pytest
import torch

from conftest import ROOT
from _util import assert_bf16_close
from oracle import restatement as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REF = os.path.join(ROOT, "baseline", "_ref")
needs_ref = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "pi3")),
                               reason="baseline/_ref is empty (baseline/install_ref.sh fills it from the reference checkout)")


def _import_ref():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import pi3.models.layers.sparse_attention as ref_sa          # noqa: F401
    return ref_sa


def _call_ref(fn, *a, **k):
    """The reference pins triton 3.3.1; with newer Triton the FIRST launch of its top-k kernel in a process
    raises "Unsupported function referenced" (a plain Python helper used inside a jitted function) and
    the same call then works.  Retry once."""
    try:
        return fn(*a, **k)
    except RuntimeError as e:
        if "Unsupported function referenced" not in str(e):
            raise
        return fn(*a, **k)


def _grid_positions(B, views, h, w, block=4):
    """(y,x) patch positions of `views` images of h x w patches in the 4x4-block-major token order of
    pi3/models/pi3_sparse.py:29-45, flattened view-major: [B, views*h*w, 2]."""
    ys, xs = torch.meshgrid(torch.arange(h), torch.arange(w), indexing="ij")
    pos = torch.stack([ys, xs], -1)                                           # [h,w,2]
    pos = pos.view(h // block, block, w // block, block, 2).permute(0, 2, 1, 3, 4).reshape(h * w, 2)
    return pos.repeat(views, 1)[None].expand(B, -1, -1).contiguous()


# --------------------------------------------------------------------------------- training size
def test_module_fwd_bwd_at_training_size():
    """B=2, 24 views of 224x224 (256 patches each): T = 6144 per sample, dim 1024, 16 heads."""
    import speed3r_b200
    torch.manual_seed(11)
    B, views, dim, heads = 2, 24, 1024, 16
    T = views * 256
    m = speed3r_b200.SparseFlashAttentionRope(dim, num_heads=heads, qkv_bias=True, qk_norm=True,
                                              rope=speed3r_b200.RoPE2D(100.0))
    with torch.no_grad():
        for name, prm in m.named_parameters():
            if name.endswith("weight") and prm.dim() == 2:
                torch.nn.init.trunc_normal_(prm, std=0.02)
            if "norm" in name:
                prm.add_(0.1 * torch.randn_like(prm))
    sd = {k: v.detach().clone().float() for k, v in m.state_dict().items()}
    m = m.to(DEV)
    m.record_idx = True
    x0 = torch.randn(B, T, dim)
    xpos = _grid_positions(B, views, 16, 16)
    dy = torch.randn(B, T, dim) * 0.1
    x = x0.to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m(x, xpos=xpos.to(DEV))
    y.float().backward(dy.to(DEV))
    idx = m.last_idx.cpu()
    p = {k: v.clone().requires_grad_(True) for k, v in sd.items()}
    xr = x0.clone().requires_grad_(True)
    y_ref, aux = R.module_forward(p, xr, xpos, heads, return_aux=True, idx_override=idx)
    y_ref.backward(dy)
    assert_bf16_close(y, y_ref, "module y", max_abs=6e-2, mean_abs=8e-3)
    assert_bf16_close(x.grad, xr.grad, "module dx", max_abs=6e-2, mean_abs=8e-3)
    for k, prm in m.named_parameters():
        assert_bf16_close(prm.grad, p[k].grad, "grad " + k, max_abs=6e-2, mean_abs=1e-2)
    # the blocks the bf16 path selected against the fp32 selection of the oracle
    _, aux0 = R.module_forward(sd, x0, xpos, heads, return_aux=True)
    same = (torch.sort(idx, -1).values == torch.sort(aux0["idx"], -1).values).float().mean().item()
    assert same > 0.9, f"only {same:.2%} of the selected blocks agree with the fp32 selection"


# ------------------------------------------------------------------ inside the reference's own code
def _swap_attention(block, rope):
    """Replace a BlockRope's reference attention by this package's class with the same weights
    (what `attn_class=speed3r_b200.SparseFlashAttentionRope` builds, pi3/models/layers/block.py:282-291)."""
    import speed3r_b200
    old = block.attn
    dim = old.qkv.in_features
    new = speed3r_b200.SparseFlashAttentionRope(dim, num_heads=old.num_heads, qkv_bias=old.qkv.bias is not None,
                                                proj_bias=old.proj.bias is not None,
                                                qk_norm=not isinstance(old.q_norm, torch.nn.Identity), rope=rope,
                                                block_size=old.block_size)
    missing = new.load_state_dict(old.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    block.attn = new.to(next(old.parameters()).device)
    return new


@needs_ref
def test_inside_reference_blockrope():
    """BlockRope(attn_class=reference SparseFlashAttentionRope) against the same block with this package's
    class: same weights, same input, the reference's own RoPE2D object (so the one-pass prologue must
    accept it) - outputs within the bf16 bound, selected blocks (nearly) identical."""
    ref_sa = _import_ref()
    from pi3.models.layers.block import BlockRope
    from pi3.models.layers.pos_embed import RoPE2D as RefRoPE2D
    from functools import partial
    import copy
    torch.manual_seed(5)
    dim, heads, views = 512, 8, 6
    rope = RefRoPE2D(freq=100.0)
    from pi3.models.dinov2.layers import Mlp
    # built the way Pi3_Sparse builds its global blocks (pi3/models/pi3_sparse.py:143-159)
    blk = BlockRope(dim=dim, num_heads=heads, mlp_ratio=4, qkv_bias=True, proj_bias=True, ffn_bias=True,
                    drop_path=0.0, norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), act_layer=torch.nn.GELU,
                    ffn_layer=Mlp, init_values=0.01, qk_norm=True, attn_class=ref_sa.SparseFlashAttentionRope,
                    rope=rope)
    with torch.no_grad():
        for name, prm in blk.named_parameters():
            if prm.dim() == 2:
                torch.nn.init.trunc_normal_(prm, std=0.05)
    blk = blk.to(DEV).eval()
    ours = copy.deepcopy(blk)
    new_attn = _swap_attention(ours, rope)
    new_attn.record_idx = True
    x = torch.randn(1, views * 256, dim, device=DEV)
    xpos = _grid_positions(1, views, 16, 16).to(DEV)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        y_ref = _call_ref(blk, x, xpos=xpos)
        assert new_attn._can_fuse_prologue(torch.empty(0), x, xpos, x.shape[1], 16, dim // heads)
        y = ours(x, xpos=xpos)
    assert_bf16_close(y, y_ref, "BlockRope output", max_abs=6e-2, mean_abs=4e-3)
    # and with gradients flowing (the separate differentiable steps)
    xg = x.clone().requires_grad_(True)
    xr = x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        yo = ours.train()(xg, xpos=xpos)
        yr = blk.train()(xr, xpos=xpos)
    dy = torch.randn_like(yo) * 0.1
    yo.backward(dy)
    yr.backward(dy)
    assert_bf16_close(yo, yr, "BlockRope output (train)", max_abs=6e-2, mean_abs=4e-3)
    assert_bf16_close(xg.grad, xr.grad, "BlockRope dx", max_abs=6e-2, mean_abs=4e-3)


@needs_ref
def test_inside_reference_pi3_sparse():
    """The unmodified reference model (its decoder cut to 4 frame + 4 global blocks to keep the test
    short; only the 1024-channel decoder matches the encoder's width), 4 views of 224x224: every global
    block's attention swapped for this package's class (same state dict).  Per global block, fed the
    reference's own input, the output matches within the bf16 bound; end to end the model outputs stay close."""
    _import_ref()
    from pi3.models.pi3_sparse import Pi3_Sparse
    import copy
    torch.manual_seed(0)
    model = Pi3_Sparse(decoder_size="large")
    model.local_decoder = torch.nn.ModuleList(list(model.local_decoder)[:4])
    model.global_decoder = torch.nn.ModuleList(list(model.global_decoder)[:4])
    with torch.no_grad():
        for name, prm in model.named_parameters():            # explicit random init: Linear weights ~ N(0, 0.02)
            if prm.dim() == 2 and "encoder" not in name:
                torch.nn.init.trunc_normal_(prm, std=0.02)
    model = model.to(DEV).eval()
    imgs = torch.rand(1, 4, 3, 224, 224, device=DEV)

    captured = []
    hooks = [blk.attn.register_forward_hook(lambda mod, args, kwargs, out: captured.append((args[0], kwargs["xpos"], out)),
                                            with_kwargs=True) for blk in model.global_decoder]
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        try:
            out_ref = model(imgs)
        except RuntimeError as e:
            if "Unsupported function referenced" not in str(e):
                raise
            captured.clear()
            out_ref = model(imgs)
    for h in hooks:
        h.remove()
    assert len(captured) == len(model.global_decoder)

    ours = copy.deepcopy(model)
    new_attns = [_swap_attention(blk, ours.rope) for blk in ours.global_decoder]
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for i, (attn, (x_in, xpos, y_ref)) in enumerate(zip(new_attns, captured)):
            y = attn(x_in, xpos=xpos)
            assert_bf16_close(y, y_ref, f"global block {i} attention", max_abs=6e-2, mean_abs=4e-3)
        out = ours(imgs)
    for key in ("local_points", "conf", "camera_poses"):
        a, b = out[key].float(), out_ref[key].float()
        rel = (a - b).norm() / b.norm().clamp_min(1e-6)
        assert rel < 5e-2, f"{key}: relative difference {rel:.3g} between the two models"


# ----------------------------------------------------------------------------- 2+ GPUs vs 1 GPU
def _partition_worker(rank, world, port, views, use_side, result):
    import torch.distributed as dist
    from speed3r_b200 import ops, seq_parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        H, D, BS, K = 16, 64, 16, 32
        T = views * 1008
        g = torch.Generator(device=dev).manual_seed(77)
        ln = lambda t: torch.nn.functional.layer_norm(t, (D,))
        q, k, v = (ln(torch.randn(1, H, T, D, device=dev, generator=g)).bfloat16() for _ in range(3))
        gate = torch.sigmoid(torch.randn(1, H, T, 2, device=dev, generator=g)).bfloat16()
        t0, t1 = seq_parallel.partition(T, BS, world, rank)
        side = torch.cuda.Stream(priority=-1) if use_side == "nccl-side" else None
        side_group = dist.new_group(list(range(world))) if use_side == "nccl-side" else None
        peer = None
        if use_side == "peer":
            shape = (1, H, (t1 - t0), D)
            peer = (seq_parallel.PeerGather(shape, torch.bfloat16, dev), seq_parallel.PeerGather(shape, torch.bfloat16, dev))
        with torch.no_grad():
            for _ in range(2):                                   # twice: the second call reuses warm communicators
                y, idx = seq_parallel.sparse_attention_partitioned(
                    *(t[:, :, t0:t1].contiguous() for t in (q, k, v, gate)), BS, K, ops.pool_tokens,
                    ops.flash_attn_topk_func, ops.sel_attn_merge_chunked, side_stream=side, side_group=side_group,
                    peer_gather=peer)
            qc, kc, vc = (ops.pool_tokens(t, BS, BS) for t in (q, k, v))
            o_c, idx_f = ops.flash_attn_topk_func(qc, kc, vc, K)
            y_f = ops.sel_attn_merge(q, k, v, idx_f, gate, o_c, BS)
            torch.cuda.synchronize()
            ok = torch.equal(y, y_f[:, t0:t1]) and torch.equal(idx, idx_f[:, :, t0 // BS:t1 // BS])
        flag = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            result.put(bool(flag.item() == 1.0))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("use_side", ["nccl", "nccl-side", "peer"])
def test_partitioned_op_equals_single_gpu(use_side):
    """Shards of the sequence-partitioned op (chunked K/V kernel input; token-level exchange by an NCCL
    all-gather, by one on a side stream with its own communicator, or by the copy engines over CUDA IPC)
    are bit-equal to the single-GPU op: 100 views, run twice so that the second exchange reuses the buffers."""
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    while (100 * 1008) % (16 * world):
        world -= 1
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + ["nccl", "nccl-side", "peer"].index(use_side)
    procs = [ctx.Process(target=_partition_worker, args=(r, world, port, 100, use_side, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(300)
    assert all(pr.exitcode == 0 for pr in procs), [pr.exitcode for pr in procs]
    assert result.get(timeout=5) is True


def _partition_grad_worker(rank, world, port, views, result):
    import torch.distributed as dist
    from speed3r_b200 import ops, seq_parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        H, D, BS, K = 4, 64, 16, 32
        T = views * 1008
        g = torch.Generator(device=dev).manual_seed(78)
        ln = lambda t: torch.nn.functional.layer_norm(t, (D,))
        q, k, v = (ln(torch.randn(1, H, T, D, device=dev, generator=g)).bfloat16() for _ in range(3))
        gate = torch.sigmoid(torch.randn(1, H, T, 2, device=dev, generator=g)).bfloat16()
        dy = torch.randn(1, T, H * D, device=dev, generator=g).bfloat16()
        t0, t1 = seq_parallel.partition(T, BS, world, rank)
        ql, kl, vl, gl = (t[:, :, t0:t1].contiguous().requires_grad_(True) for t in (q, k, v, gate))
        y, idx = seq_parallel.sparse_attention_partitioned_grad(ql, kl, vl, gl, BS, K, ops.pool_tokens,
                                                                ops.flash_attn_topk_func, ops.sel_attn_merge)
        y.backward(dy[:, t0:t1].contiguous())
        qf, kf, vf, gf = (t.clone().requires_grad_(True) for t in (q, k, v, gate))
        qc, kc, vc = (ops.pool_tokens(t, BS, BS) for t in (qf, kf, vf))
        o_c, idx_f = ops.flash_attn_topk_func(qc, kc, vc, K)
        y_f = ops.sel_attn_merge(qf, kf, vf, idx_f, gf, o_c, BS)
        y_f.backward(dy)
        torch.cuda.synchronize()
        ok = torch.equal(y.detach(), y_f.detach()[:, t0:t1]) and torch.equal(idx, idx_f[:, :, t0 // BS:t1 // BS])
        # dq, dgate: the same kernels on the same rows; dk, dv: partial sums rounded to bf16 before the reduction
        for name, a, b, tol in (("dq", ql.grad, qf.grad[:, :, t0:t1], 0.0), ("dgate", gl.grad, gf.grad[:, :, t0:t1], 0.0),
                                ("dk", kl.grad, kf.grad[:, :, t0:t1], 3e-2), ("dv", vl.grad, vf.grad[:, :, t0:t1], 3e-2)):
            diff = (a.float() - b.float()).abs().max().item()
            scale = max(1.0, b.float().abs().max().item())
            if diff > tol * scale:
                print(f"rank {rank}: {name} differs by {diff} (scale {scale})", flush=True)
                ok = False
        flag = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            result.put(bool(flag.item() == 1.0))
    finally:
        dist.destroy_process_group()


def test_partitioned_op_gradients_match_single_gpu():
    """Forward + backward of the sequence-partitioned op on 2+ GPUs against the single-GPU op on the global
    tensors: outputs, tables, dQ and dgate bit-equal; dK and dV (reduce-scattered bf16 partial sums) within
    bf16 rounding of the single-GPU gradients."""
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    while (20 * 1008) % (16 * world):
        world -= 1
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + 7
    procs = [ctx.Process(target=_partition_grad_worker, args=(r, world, port, 20, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(300)
    assert all(pr.exitcode == 0 for pr in procs), [pr.exitcode for pr in procs]
    assert result.get(timeout=5) is True


def _ddp_worker(rank, world, port, result):
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP
    import speed3r_b200
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, views, hw, dim, heads = 2, 24, 16, 1024, 16            # 24 views of 224 x 224: 16 x 16 patches each
        T = views * hw * hw
        torch.manual_seed(11)                                     # the same weights on every rank
        rope = speed3r_b200.RoPE2D(100.0)
        mod = speed3r_b200.SparseFlashAttentionRope(dim, num_heads=heads, qkv_bias=True, qk_norm=True, rope=rope).to(dev)
        pos = _grid_positions(B, views, hw, hw).to(dev)
        def batch(seed):
            g = torch.Generator(device=dev).manual_seed(seed)
            return (torch.randn(B, T, dim, device=dev, generator=g) * 0.5, torch.randn(B, T, dim, device=dev, generator=g))
        # every rank's gradient on its own batch without DDP, averaged over ranks by hand ...
        grads = []
        for r in range(world):
            x, dy = batch(100 + r)
            mod.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = mod(x, xpos=pos)
            y.float().backward(dy)
            grads.append([p.grad.detach().clone() for p in mod.parameters()])
        mean = [sum(gs) / world for gs in zip(*grads)]
        # ... against one DDP step in which every rank sees only its own batch
        mod.zero_grad(set_to_none=True)
        ddp = DDP(mod, device_ids=[rank])
        x, dy = batch(100 + rank)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = ddp(x, xpos=pos)
        y.float().backward(dy)
        torch.cuda.synchronize()
        ok = True
        for (name, p), m in zip(mod.named_parameters(), mean):
            err = (p.grad - m).abs().max().item()
            if err > 1e-3 * max(1.0, m.abs().max().item()):
                print(f"rank {rank}: {name} grad differs by {err}", flush=True)
                ok = False
        flag = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            result.put(bool(flag.item() == 1.0))
    finally:
        dist.destroy_process_group()


def test_data_parallel_training_step():
    """The reference's training configuration (B=2 per GPU, 24 views of 224 x 224 -> 6144 tokens per sample,
    DistributedDataParallel): one forward + backward of the module under DDP gives every rank the mean of
    the per-rank gradients (the kernels are deterministic, so the only difference is the all-reduce's order)."""
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + 9
    procs = [ctx.Process(target=_ddp_worker, args=(r, world, port, result)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(600)
    assert all(pr.exitcode == 0 for pr in procs), [pr.exitcode for pr in procs]
    assert result.get(timeout=5) is True
