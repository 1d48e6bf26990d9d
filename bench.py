#!/usr/bin/env python
"""Benchmark of the sparse global-attention layer op at 1000 views (the reference's headline
setting), on synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--views V] [--mode fwd|fwdbwd]

One step = one pass of the op over one 1000-view sequence: pool q,k,v (16/16) -> compression
attention with fused top-32 -> selection attention over the 32 selected 16-token blocks with the
gated merge fused.  Inputs: q,k,v ~ N(0,1) after a per-head LayerNorm, bf16, [1,16,T,64] with
T = views*1008; gate = sigmoid(N(0,1)).  The metric is effective sparse TFLOP/s
(F = 4*Nq*Nc*d*H + 4*T*K*Bs*d*H per step, forward; x3.5 with the backward).

N > 1 (launched with torch.distributed.run): the sequence is partitioned by query blocks over the
ranks; pooled and token-level K/V are all-gathered (NCCL).  Total work is fixed -> strong scaling.
Every rank draws the GLOBAL tensors from one seed and keeps its slice, so that (outside the timed
region) each rank can run the single-GPU op on the global tensors and check that its shard of the
partitioned result is bit-identical (`parity` in the JSON line).

At N = 1 the line also carries `triton_baseline`: the reference's own Triton kernels (unmodified, from
baseline/_ref, installed by baseline/install_ref.sh) timed on the same GPU and the same tensors, and
the dense `F.scaled_dot_product_attention` time at the same sequence length.

--impl reference times the CPU restatement of the reference's algorithm (the reference itself is
Python + Triton and is not present on the benchmark machine) on a bounded sample of the same
workload, using all host threads.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, D, BS, TOPK, TOK_PER_VIEW = 16, 64, 16, 32, 1008


def flops_fwd(T, Nq_rows=None, heads=H):
    """Effective sparse flops of one forward of the op (optionally for a subset of query blocks)."""
    nq = T // BS if Nq_rows is None else Nq_rows
    nc = T // BS
    f_cmp = 4.0 * nq * nc * D * heads
    f_sel = 4.0 * (nq * BS) * (TOPK * BS) * D * heads
    return f_cmp, f_sel


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm_gbs=j["hbm_gbs"], tflops=j["bf16_tflops_sustained"], tflops_burst=j["bf16_tflops"], src="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, tflops_burst=1590.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the GPU runs the workload.

    nvidia-smi needs about a second before its first row, so the sampler is started before the warm-up and
    every row carries its arrival time; `stop(t0, t1)` reports the rows that fell inside the timed region
    and, when that region was too short to catch two, the rows of the whole loaded window
    (`hold()` keeps the same step running, untimed, until enough rows have arrived)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def count_since(self, t0):
        return sum(1 for t, _ in self.rows if t >= t0)

    def stop(self, t0, t1, t_hold):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        inside = [r for t, r in self.rows if t0 <= t <= t1]
        window = "timed region"
        if len(inside) < 2:
            inside = [r for t, r in self.rows if t0 <= t <= t_hold]
            window = "timed region + the same step repeated untimed right after it"
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
                for n, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        busy = [x for x in sm if mx and x > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "window": window}


# --------------------------------------------------------------------------------------------------
# CPU arm: the oracle restatement on a bounded sample of the same workload
# --------------------------------------------------------------------------------------------------
def cpu_sample(views, seconds_hint=20.0):
    """One head, the first `nqb` query blocks against ALL pooled keys / token blocks of the head."""
    import torch
    from oracle import restatement as R
    torch.set_num_threads(os.cpu_count() or 1)
    T = views * TOK_PER_VIEW
    nc = T // BS
    nqb = max(8, min(nc, int(2.0e10 / (4.0 * nc * D + 4.0 * BS * TOPK * BS * D))))   # ~20 Gflop of work
    g = torch.Generator().manual_seed(0)
    ln = lambda t: torch.nn.functional.layer_norm(t, (D,))
    q = ln(torch.randn(1, 1, nqb * BS, D, generator=g)).bfloat16().float()
    k = ln(torch.randn(1, 1, T, D, generator=g)).bfloat16().float()
    v = ln(torch.randn(1, 1, T, D, generator=g)).bfloat16().float()
    gate = torch.sigmoid(torch.randn(1, 1, nqb * BS, 2, generator=g))

    def step():
        q_c, k_c, v_c = R.pool_tokens(q, BS, BS), R.pool_tokens(k, BS, BS), R.pool_tokens(v, BS, BS)
        o_c, _, idx = R.cmp_attn_topk(q_c, k_c, v_c, TOPK, row_chunk=512)
        o_s, _ = R.sel_attn(q, k, v, idx, BS, qblock_chunk=256)
        return R.gated_merge(gate, o_c, o_s, BS)

    f_cmp, f_sel = flops_fwd(T, Nq_rows=nqb, heads=1)
    sample = (f"1 head, first {nqb} of {nc} query blocks against all {nc} pooled keys and the full K/V of the "
              f"{views}-view sequence, fp32 torch on {torch.get_num_threads()} threads")
    return step, f_cmp + f_sel, sample, torch.get_num_threads()


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, fl, sample, cores = cpu_sample(args.views)
    for _ in range(max(1, min(args.warmup, 1))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = fl / dt / 1e12
    line = dict(metric="sparse_attn_layer_effective_tflops", value=val, unit="TFLOP/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=dt * 1e3, higher_is_better=True,
                scaling="strong", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=workload_config(args),
                cpu_baseline=dict(value=val, unit="TFLOP/s", cores=cores, kind="port", sample=sample),
                e2e=dict(value=val, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line))


def workload_config(args):
    T = args.views * TOK_PER_VIEW
    return {"workload": f"sparse global-attention op, {args.mode}, {args.views} views x {TOK_PER_VIEW} tokens "
                        f"(T={T}), H={H}, d={D}, pool {BS}/{BS}, select block {BS}, top-{TOPK}, {getattr(args, 'inputs', 'iid')} inputs",
            "tokens": T, "views": args.views, "mode": args.mode,
            "parallelism": (f"sp{args.gpus}, token K/V exchange: " + ("peer pull kernel over CUDA IPC" if getattr(args, "gather", "nccl") == "peer"
                                                                       else "NCCL all-gather on a side stream")) if args.gpus > 1 else "single",
            "l2": "inputs (q,k,v: 3 x %.1f GB) larger than the 126 MB L2" % (T * H * D * 2 / 1e9)}


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def make_inputs(args, T, dev):
    """q, k, v [1,H,T,64] bf16 after a per-head LayerNorm and gate [1,H,T,2], from ONE seed (the same
    tensors on every rank).  `structured`: every token's key/query is the sum of a component shared by
    its view, a component shared by its patch position across views and noise, mixed through a rank-16
    map, so that neighbouring query blocks select overlapping key blocks (as real multi-view features do)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(1234)
    ln = lambda t: torch.nn.functional.layer_norm(t, (D,))
    if args.inputs == "iid":
        q, k, v = (ln(torch.randn(1, H, T, D, device=dev, generator=g)).bfloat16() for _ in range(3))
    else:
        views, tok = T // TOK_PER_VIEW, TOK_PER_VIEW
        def structured():
            r = 16
            view = torch.randn(1, H, views, 1, r, device=dev, generator=g)
            patch = torch.randn(1, H, 1, tok, r, device=dev, generator=g)
            mix = torch.randn(1, H, r, D, device=dev, generator=g) / 4.0
            low = ((view + patch).reshape(1, H, T, r) @ mix)
            return ln(low + 0.5 * torch.randn(1, H, T, D, device=dev, generator=g)).bfloat16()
        q, k = structured(), structured()
        v = ln(torch.randn(1, H, T, D, device=dev, generator=g)).bfloat16()
    gate = torch.sigmoid(torch.randn(1, H, T, 2, device=dev, generator=g)).bfloat16()
    return q, k, v, gate


def triton_baseline(q, k, v, views):
    """The reference's own kernels (flash_attention_topk.forward_with_topk :156-200 and
    topk_blocksparse_attention._topk_blocksparse_attention_fwd :852-904) from baseline/_ref, unmodified,
    on the same device and tensors: pooled q,k,v -> compression attention + top-k -> selection attention.
    Returns a dict for the JSON line (`unavailable` with the reason when it cannot run)."""
    import torch
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "pi3")):
        return {"unavailable": "baseline/_ref is empty (run baseline/install_ref.sh where the reference checkout is)"}
    try:
        if ref not in sys.path:
            sys.path.insert(0, ref)
        import triton
        from pi3.models.sparse_attn.flash_attention_topk import forward_with_topk
        from pi3.models.sparse_attn.topk_blocksparse_attention import _topk_blocksparse_attention_fwd
        from speed3r_b200 import ops
        qc, kc, vc = (ops.pool_tokens(t, BS, BS) for t in (q, k, v))
        ev = lambda: torch.cuda.Event(enable_timing=True)

        def timed(fn, warm, reps):
            for i in range(warm):
                try:
                    fn()
                except RuntimeError:
                    if i > 0:            # the first JIT of a kernel can fail on a helper reference and pass on retry
                        raise
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            for _ in range(reps):
                out = fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps, out

        warm = 10
        t_cmp, (o_c, _, idx, _) = timed(lambda: forward_with_topk(qc, kc, vc, TOPK), warm, 3)
        t_sel, (o_s, _) = timed(lambda: _topk_blocksparse_attention_fwd(q, k, v, idx, BS, 1.0 / math.sqrt(D)), warm, 3)
        o2, idx2 = ops.flash_attn_topk_func(qc, kc, vc, TOPK)
        o3 = ops.topk_blocksparse_attention(q, k, v, idx, BS)
        torch.cuda.synchronize()
        return {"what": "reference Triton kernels, unmodified: forward_with_topk + _topk_blocksparse_attention_fwd "
                        "(pooling by this library; the merge is not included)",
                "triton": triton.__version__, "views": views, "warmup": warm, "reps": 3,
                "cmp_attn_topk_ms": t_cmp, "sel_attn_ms": t_sel, "total_ms": t_cmp + t_sel,
                "idx_mismatch_fraction_vs_ours": (idx != idx2).float().mean().item(),
                "o_c_max_abs_diff_vs_ours": (o_c.float() - o2.float()).abs().max().item(),
                "o_s_max_abs_diff_vs_ours": (o_s.float() - o3.float()).abs().max().item()}
    except Exception as e:      # Triton failing to compile or run these kernels on this GPU is a result, not a crash
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def dense_baseline(q, k, v):
    """Dense attention over the same sequence with the library flash kernel (F.scaled_dot_product_attention)."""
    import torch
    try:
        f = lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v)
        f()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        f()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        T = q.shape[2]
        return {"what": "F.scaled_dot_product_attention, same q,k,v, 1 iteration after 1 warm-up", "ms": ms,
                "tflops": 4.0 * T * T * D * H / ms / 1e9}
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def run_model(args):
    """Forward of the reference's Pi3_Sparse (unmodified code from baseline/_ref, random weights, 392x504
    images: 28x36 patches = 1008 tokens per view) with the global blocks' attention swapped for this
    package's class.  With N > 1 every rank holds views/N views: encoder, frame blocks, MLPs and heads
    are per view and need no communication (pi3/models/pi3_sparse.py:214-321); the global attention runs
    sequence-partitioned (speed3r_b200.seq_parallel)."""
    import torch
    import torch.distributed as dist
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "pi3")):
        print(json.dumps({"metric": "pi3_sparse_forward_views_per_s", "unavailable":
                          "baseline/_ref is empty (run baseline/install_ref.sh where the reference checkout is)"}))
        return
    sys.path.insert(0, ref)
    import speed3r_b200
    from speed3r_b200 import seq_parallel
    from pi3.models.pi3_sparse import Pi3_Sparse
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.model_attn == "reference" and world > 1:
        raise SystemExit("the reference attention is single-GPU")
    if args.views % world:
        raise SystemExit("--views must be a multiple of --gpus")
    torch.manual_seed(0)                                   # the same weights on every rank
    model = Pi3_Sparse()
    with torch.no_grad():
        for name, prm in model.named_parameters():         # explicit init: Linear weights trunc-normal(0.02), biases 0,
            if prm.dim() == 2:                             # the gates keep their (-1,+1) bias
                torch.nn.init.trunc_normal_(prm, std=0.02)
            elif prm.dim() == 1 and name.endswith(".bias") and ".gate." not in name:
                prm.zero_()
    model = model.to(dev).eval()
    attns = []
    if args.model_attn == "ours":
        sp = seq_parallel.SequenceParallel(gather=args.gather) if world > 1 else None
        for blk in model.global_decoder:
            old = blk.attn
            new = speed3r_b200.SparseFlashAttentionRope(old.qkv.in_features, num_heads=old.num_heads, qkv_bias=True,
                                                        proj_bias=True, qk_norm=True, rope=model.rope,
                                                        block_size=old.block_size)
            new.load_state_dict(old.state_dict())
            new.seq_parallel = sp
            blk.attn = new.to(dev)
    attns = [blk.attn for blk in model.global_decoder]
    vl = args.views // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    imgs = torch.rand(1, vl, 3, 392, 504, device=dev, generator=g)
    marks = []
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def before(mod, inputs):
        marks.append([ev(), ev()])
        marks[-1][0].record()

    def after(mod, inputs, output):
        marks[-1][1].record()

    for a_ in attns:
        a_.register_forward_pre_hook(before)
        a_.register_forward_hook(after)

    def fwd():
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            try:
                return model(imgs)
            except RuntimeError as e:       # newer Triton than the reference pins: its first launch can fail once
                if "Unsupported function referenced" not in str(e):
                    raise
                return model(imgs)

    warm = max(1, min(args.warmup, 2))
    for _ in range(warm):
        fwd()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    marks.clear()
    steps = max(1, min(args.steps, 3))
    a, b = ev(), ev()
    a.record()
    for _ in range(steps):
        out = fwd()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    attn_ms = sum(m[0].elapsed_time(m[1]) for m in marks) / steps
    if world > 1:
        t = torch.tensor([ms, attn_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, attn_ms = t[0].item(), t[1].item()
    finite = bool(torch.isfinite(out["points"]).all().item())
    if rank == 0:
        print(json.dumps(dict(
            metric="pi3_sparse_forward_views_per_s", value=args.views / (ms * 1e-3), unit="views/s", n_gpus=world,
            steps=steps, warmup=warm, ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None,
            dtype="bf16", data="synthetic",
            config={"workload": f"Pi3_Sparse forward (reference model code, random weights), {args.views} views of 392x504, "
                                f"global attention: {'this library' if args.model_attn == 'ours' else 'reference Triton module'}",
                    "views": args.views, "tokens": args.views * TOK_PER_VIEW,
                    "parallelism": f"views sharded over {world} GPUs, global attention sequence-partitioned ({args.gather})"
                                   if world > 1 else "single"},
            model={"global_attention_ms": attn_ms, "global_attention_share": attn_ms / ms,
                   "global_blocks": len(attns), "outputs_finite": finite})))
    if world > 1:
        dist.destroy_process_group()


def run_train_step(args):
    """One data-parallel training step of the attention module at the reference's training size (BASELINE
    config 5: B=2 per GPU, 24 views of 224x224 -> 6144 tokens per sample, dim 1024, 16 heads, bf16 autocast,
    DistributedDataParallel as in trainers/base_trainer_accelerate.py:102): forward, backward with the
    gradient all-reduce, and an AdamW update of the module's parameters.  Weak scaling (the per-GPU batch is fixed)."""
    import torch
    import torch.distributed as dist
    import speed3r_b200
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B, views, hw, dim = 2, 24, 16, H * D
    T = views * hw * hw
    torch.manual_seed(0)
    mod = speed3r_b200.SparseFlashAttentionRope(dim, num_heads=H, qkv_bias=True, proj_bias=True, qk_norm=True,
                                                rope=speed3r_b200.RoPE2D(100.0)).to(dev)
    net = torch.nn.parallel.DistributedDataParallel(mod, device_ids=[local_rank]) if world > 1 else mod
    opt = torch.optim.AdamW(mod.parameters(), lr=1e-4)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(B, T, dim, device=dev, generator=g) * 0.5
    dy = torch.randn(B, T, dim, device=dev, generator=g) * 0.1
    tok = torch.arange(T, device=dev) % (hw * hw)
    xpos = torch.stack((tok // hw, tok % hw), -1)[None].expand(B, -1, -1).contiguous()

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = net(x, xpos=xpos)
        y.float().backward(dy)
        opt.step()

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    status = _lib_status()
    if rank == 0:
        print(json.dumps(dict(
            metric="attention_module_train_tokens_per_s", value=world * B * T / (ms * 1e-3), unit="tokens/s", n_gpus=world,
            steps=args.steps, warmup=max(3, args.warmup), ms_per_step=ms, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="bf16", data="synthetic",
            config={"workload": "SparseFlashAttentionRope forward + backward + AdamW step, B=2 per GPU, 24 views of 224x224 "
                                "(T=6144 per sample), dim 1024, 16 heads", "global_batch": world * B, "tokens_per_sample": T,
                    "parallelism": f"ddp{world}" if world > 1 else "single"},
            device_status=status)))
    if world > 1:
        dist.destroy_process_group()


def run_extension(args):
    """The op at BASELINE's other setting - keys/values pooled with kernel 32 and stride 16, selection blocks of
    64 tokens, top-16 - forward on one GPU, same inputs as the default workload.  Queries are pooled per
    selection block and the table ranks blocks by the softmax mass of their three inner compressed keys (the
    reference has no such mode: its three sizes are equal; the oracle's `block_rank_scores` is the definition)."""
    import torch
    from speed3r_b200 import ops, _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Lc, Sc, Bs, K = 32, 16, 64, 16
    T = args.views * TOK_PER_VIEW
    T -= T % Bs
    q, k, v, gate = make_inputs(args, T, dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    marks = []

    def step():
        e = [ev() for _ in range(4)]
        e[0].record()
        q_c, k_c, v_c = ops.pool_tokens(q, Bs, Bs), ops.pool_tokens(k, Lc, Sc), ops.pool_tokens(v, Lc, Sc)
        e[1].record()
        o_c, idx = ops.flash_attn_blocktopk_func(q_c, k_c, v_c, K, Bs // Sc, (Bs - Lc) // Sc + 1)
        e[2].record()
        y = ops.sel_attn_merge(q, k, v, idx, gate, o_c, Bs)
        e[3].record()
        marks.append(e)
        return y

    with torch.no_grad():
        for _ in range(max(3, args.warmup)):
            step()
        torch.cuda.synchronize()
        marks.clear()
        a, b = ev(), ev()
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    avg = lambda i: sum(m[i].elapsed_time(m[i + 1]) for m in marks) / len(marks)
    Nq, Nc = T // Bs, (T - Lc) // Sc + 1
    f_cmp, f_sel = 4.0 * Nq * Nc * D * H, 4.0 * T * K * Bs * D * H
    print(json.dumps(dict(
        metric="sparse_attn_layer_effective_tflops", value=(f_cmp + f_sel) / (ms * 1e-3) / 1e12, unit="TFLOP/s", n_gpus=1,
        steps=args.steps, warmup=max(3, args.warmup), ms_per_step=ms, higher_is_better=True, scaling="strong",
        vs_baseline=None, dtype="bf16", data="synthetic",
        config={"workload": f"sparse global-attention op, fwd, {args.views} views x {TOK_PER_VIEW} tokens (T={T}), H={H}, d={D}, "
                            f"pool {Lc}/{Sc}, select block {Bs}, top-{K}, blocks ranked by probability mass, {args.inputs} inputs",
                "tokens": T, "views": args.views, "parallelism": "single"},
        kernels={"pool_ms": avg(0), "cmp_attn_blocktopk_ms": avg(1), "sel_attn_merge_ms": avg(2),
                 "cmp_tflops": f_cmp / avg(1) / 1e9, "sel_tflops": f_sel / avg(2) / 1e9},
        device_status=_lib.device_status())))


def _lib_status():
    from speed3r_b200 import _lib
    return _lib.device_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--views", type=int, default=1000)
    ap.add_argument("--mode", default="fwd", choices=["fwd", "fwdbwd"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--module", action="store_true", help="also time the whole attention module at this size")
    ap.add_argument("--inputs", default="iid", choices=["iid", "structured"],
                    help="iid: q,k,v ~ N(0,1) per token; structured: keys/queries = low-rank view + patch components")
    ap.add_argument("--model", action="store_true",
                    help="time the forward of the reference's own Pi3_Sparse (from baseline/_ref) with this package's "
                         "attention class swapped in; prints a line of its own (metric pi3_sparse_forward_views_per_s)")
    ap.add_argument("--model-attn", default="ours", choices=["ours", "reference"],
                    help="--model: which attention class the global blocks use (reference = its Triton module, 1 GPU only)")
    ap.add_argument("--gather", default="nccl", choices=["peer", "nccl"],
                    help="N > 1: token-level K/V exchange by an NCCL all-gather on a side stream (default, measured "
                         "fastest) or by this library's peer pull kernel over CUDA IPC")
    ap.add_argument("--train-step", action="store_true",
                    help="time one data-parallel training step of the attention module at the reference's training "
                         "size (B=2 per GPU, T=6144); prints a line of its own (metric attention_module_train_tokens_per_s)")
    ap.add_argument("--setting", default="reference", choices=["reference", "extension"],
                    help="reference: pool 16/16, blocks of 16, top-32 (the reference's only setting); extension: pool 32/16, "
                         "blocks of 64, top-16 with block ranking by probability mass (1 GPU, forward; a line of its own)")
    ap.add_argument("--no-triton-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps > 5:
            args.steps = 5
        run_reference_arm(args)
        return
    if args.model:
        run_model(args)
        return
    if args.train_step:
        run_train_step(args)
        return
    if args.setting == "extension":
        run_extension(args)
        return

    import torch
    import torch.distributed as dist
    from speed3r_b200 import _lib, ops, seq_parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    args.warmup = max(args.warmup, 3)

    T = args.views * TOK_PER_VIEW
    tok0, tok1 = seq_parallel.partition(T, BS, world, rank)
    Tl = tok1 - tok0
    qg, kg, vg, gateg = make_inputs(args, T, dev)           # GLOBAL tensors, identical on every rank
    if world > 1:
        q, k, v, gate = (t[:, :, tok0:tok1].contiguous() for t in (qg, kg, vg, gateg))
    else:
        q, k, v, gate = qg, kg, vg, gateg
    g = torch.Generator(device=dev).manual_seed(99)
    bwd = args.mode == "fwdbwd"
    # fwdbwd at N > 1: the differentiable partitioned op (dense gathered K/V; dK/dV reduce-scattered in the backward)
    dy = torch.randn(1, Tl, H * D, device=dev, generator=g).bfloat16() if bwd else None
    # high priority: the all-gather's few CTAs must not queue behind the compression kernel, which fills every SM
    side = torch.cuda.Stream(priority=-1) if world > 1 else None
    side_group = dist.new_group(list(range(world))) if world > 1 else None     # own communicator for the large all-gather
    peer = None
    if world > 1 and args.gather == "peer":
        peer = (seq_parallel.PeerGather((1, H, Tl, D), torch.bfloat16, dev),
                seq_parallel.PeerGather((1, H, Tl, D), torch.bfloat16, dev))

    ev = lambda: torch.cuda.Event(enable_timing=True)
    marks = []

    def step_partitioned(q_, k_, v_, g_, record=False, with_idx=False):
        """N > 1: this rank's query blocks; events around the two attention kernels when recording."""
        e = [ev() for _ in range(4)] if record else None

        def cmp_fn(a, b, c, kk):
            if record: e[0].record()
            r = ops.flash_attn_topk_func(a, b, c, kk)
            if record: e[1].record()
            return r

        def sel_fn(a, b, c, i, gt, oc, bs):
            if record: e[2].record()
            r = ops.sel_attn_merge_chunked(a, b, c, i, gt, oc, bs)
            if record: e[3].record()
            return r

        y, idx_ = seq_parallel.sparse_attention_partitioned(q_, k_, v_, g_, BS, TOPK, ops.pool_tokens, cmp_fn, sel_fn,
                                                            side_stream=side, side_group=side_group, peer_gather=peer)
        if record:
            marks.append(e)
        return (y, idx_) if with_idx else y

    def step(record=False):
        """Returns y; with record=True also appends per-kernel CUDA events."""
        if world > 1 and bwd:
            ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
            y, _ = seq_parallel.sparse_attention_partitioned_grad(ql, kl, vl, gate, BS, TOPK, ops.pool_tokens,
                                                                  ops.flash_attn_topk_func, ops.sel_attn_merge)
            y.backward(dy)
            return y
        if world > 1:
            return step_partitioned(q, k, v, gate, record)
        if bwd:
            ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        else:
            ql, kl, vl = q, k, v
        e = [ev() for _ in range(4)] if record else None
        if record: e[0].record()
        qc, kc, vc = (ops.pool_tokens(t, BS, BS) for t in (ql, kl, vl))
        if record: e[1].record()
        o_c, idx = ops.flash_attn_topk_func(qc, kc, vc, TOPK)
        if record: e[2].record()
        y = ops.sel_attn_merge(ql, kl, vl, idx, gate, o_c, BS)
        if record:
            e[3].record()
            marks.append(e)
        if bwd:
            y.backward(dy)
        return y

    ctx = torch.enable_grad() if bwd else torch.no_grad()
    with ctx:
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e_ = ev(), ev()
        t0 = time.time()
        s.record()
        for _ in range(args.steps):
            step(record=True)
        e_.record()
        torch.cuda.synchronize()
        t1 = time.time()
        if world > 1:
            dist.barrier()
        # a timed region shorter than the sampler's period: keep the same load on, untimed, until it has rows
        hold = torch.zeros(1, device=dev)
        while True:
            if rank == 0:
                need = sampler.proc is not None and sampler.count_since(t0) < 3 and time.time() - t1 < 3.0
                hold.fill_(1.0 if need else 0.0)
            if world > 1:
                dist.broadcast(hold, 0)
            if hold.item() == 0.0:
                break
            step()
            torch.cuda.synchronize()
        clocks = sampler.stop(t0, t1, time.time()) if rank == 0 else None
        ms = s.elapsed_time(e_) / args.steps
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = tms.item()
    status = _lib.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status}: a kernel gave up a bounded wait")

    # N > 1, outside the timed region: this rank's shard of the partitioned result against the single-GPU
    # op run here on the global tensors.  The chunked-K/V kernel is bit-identical to the dense one, so
    # equality is the bar, for the output and for the selected-block table.
    parity = None
    if world > 1 and not bwd and not args.no_parity:
        with torch.no_grad():
            y_sh, idx_sh = step_partitioned(q, k, v, gate, with_idx=True)
            qc_, kc_, vc_ = (ops.pool_tokens(t, BS, BS) for t in (qg, kg, vg))
            o_c_, idx_f = ops.flash_attn_topk_func(qc_, kc_, vc_, TOPK)
            y_f = ops.sel_attn_merge(qg, kg, vg, idx_f, gateg, o_c_, BS)
            ok_y = torch.equal(y_sh, y_f[:, tok0:tok1])
            ok_i = torch.equal(idx_sh, idx_f[:, :, tok0 // BS:tok1 // BS])
            flags = torch.tensor([1.0 if ok_y else 0.0, 1.0 if ok_i else 0.0], device=dev)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            del y_sh, idx_sh, qc_, kc_, vc_, o_c_, idx_f, y_f
        parity = {"ok": bool(flags[0].item() == 1.0 and flags[1].item() == 1.0),
                  "y_bit_equal": bool(flags[0].item() == 1.0), "idx_bit_equal": bool(flags[1].item() == 1.0),
                  "checked": f"on every one of the {world} ranks: y and idx shards of the partitioned op == the same "
                             f"rows of the single-GPU op on the global tensors ({args.views} views)"}
    tri = dense = None
    if world == 1 and not bwd and not args.no_triton_baseline:
        with torch.no_grad():
            tri = triton_baseline(q, k, v, args.views)
            dense = dense_baseline(q, k, v)
        torch.cuda.empty_cache()
    del qg, kg, vg, gateg

    f_cmp, f_sel = flops_fwd(T)
    ftot = (f_cmp + f_sel) * (3.5 if bwd else 1.0)
    value = ftot / (ms * 1e-3) / 1e12
    peaks = load_peaks()

    # per-kernel averages (single GPU): pooling, compression attention + top-k, selection + merge
    roof, kern = None, None
    if world > 1 and marks and rank == 0:
        # rank 0's share of the work: Nq/world query rows against all Nc pooled keys
        avg = lambda i: sum(m[i].elapsed_time(m[i + 1]) for m in marks) / len(marks)
        t_cmp, t_sel = avg(0), avg(2)
        ach = f_cmp / world / t_cmp / 1e9
        kern = {"cmp_attn_topk_ms": t_cmp, "sel_attn_merge_ms": t_sel, "rank": 0,
                "cmp_tflops_per_gpu": ach, "sel_tflops_per_gpu": f_sel / world / t_sel / 1e9,
                # what of the step is not the two attention kernels on rank 0: pooling, the pooled all-gathers
                # the compression kernel waits for, and the part of the token K/V all-gather it does not cover
                "exposed_comm_ms": ms - t_cmp - t_sel}
        roof = {"kernel": "cmp_fwd_kernel (compression attention + top-k), rank 0", "bound": "tensor", "achieved": ach,
                "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"], "traffic": None,
                "peak_source": f"{peaks['src']} sustained bf16 (kernel timed inside a long step)"}
    if world == 1 and marks:
        avg = lambda i: sum(m[i].elapsed_time(m[i + 1]) for m in marks) / len(marks)
        t_pool, t_cmp, t_sel = avg(0), avg(1), avg(2)
        pool_bytes = 3 * T * H * D * 2 + 3 * (T // BS) * H * D * 2
        sel_bytes = (T // BS) * H * TOPK * BS * D * 4 + 2 * T * H * D * 2 + T * H * 2 * 2
        kern = {"pool_ms": t_pool, "cmp_attn_topk_ms": t_cmp, "sel_attn_merge_ms": t_sel,
                "pool_gbs": pool_bytes / t_pool / 1e6, "pool_frac_hbm": pool_bytes / t_pool / 1e6 / peaks["hbm_gbs"],
                "cmp_tflops": f_cmp / t_cmp / 1e9, "sel_gather_gbs": sel_bytes / t_sel / 1e6,
                "sel_tflops": f_sel / t_sel / 1e9}
        # the gather figure counts every selected block as if it came from DRAM; L2 serves part of it.  DRAM
        # traffic of this kernel measured with ncu on this workload (one-pass capture of one launch):
        # 64.21 GB read + 2.07 GB written per launch at 1000 views (not proportional to views: L2 hit rate changes)
        if args.views == 1000:
            kern["sel_dram_gbs"] = 66.27e9 / t_sel / 1e6
            kern["sel_frac_hbm"] = kern["sel_dram_gbs"] / peaks["hbm_gbs"]
        ach = f_cmp / t_cmp / 1e9
        # DRAM traffic of one launch: an ncu capture of an earlier version of the kernel on this workload
        # (1000 views: dram__bytes_read.sum 392.4 MB + dram__bytes_write.sum 235.1 MB).  It equals the
        # algorithmic bytes (pooled q,k,v read once: 387 MB; o_c, lse and the table written once: 262 MB) and
        # grows with views.  The capture of the current kernel was taken at 100 views (38.8 MB read = the
        # inputs once; the outputs were still in L2 when the kernel ended), so the full-size figure is kept.
        traffic = 627.5e6 * (args.views / 1000.0)
        roof = {"kernel": "cmp_fwd_kernel (compression attention + top-k)", "bound": "tensor", "achieved": ach,
                "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"], "traffic": traffic,
                "traffic_unit": "bytes/launch (ncu dram read+write of a 1000-view capture, = the algorithmic bytes, scaled by views)",
                "peak_source": f"{peaks['src']} sustained bf16 (kernel timed inside a long step)"}

    # end to end through the public op functions with HOST buffers (pinned), copies inside the timing
    e2e = None
    if not args.no_e2e and not bwd:
        # every rank moves its own shard: pinned host -> device, run, result back to pinned host
        hq, hk, hv, hg = (t.cpu().pin_memory() for t in (q, k, v, gate))
        hy = torch.empty(1, Tl, H * D, dtype=torch.bfloat16).pin_memory()
        if world > 1:
            dq_, dk_, dv_, dg_ = (torch.empty_like(t) for t in (q, k, v, gate))

        pipe = None
        if world == 1:
            from speed3r_b200.host_pipeline import HostPipeline
            pipe = HostPipeline(H, T, D, BS, TOPK, device=dev)

        def e2e_step():
            if pipe is not None:          # copies overlapped with the kernels on three streams
                pipe(hq, hk, hv, hg, hy)
                return
            dq_.copy_(hq, non_blocking=True); dk_.copy_(hk, non_blocking=True)
            dv_.copy_(hv, non_blocking=True); dg_.copy_(hg, non_blocking=True)
            y = step_partitioned(dq_, dk_, dv_, dg_)
            hy.copy_(y, non_blocking=True)

        with torch.no_grad():
            e2e_step()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            n = max(2, min(args.steps, 5))
            s2, e2 = ev(), ev()
            s2.record()
            for _ in range(n):
                e2e_step()
            e2.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ems = s2.elapsed_time(e2) / n
        if world > 1:
            tms = torch.tensor([ems], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            ems = tms.item()
        e2e = {"value": (f_cmp + f_sel) / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ems,
               "h2d_bytes_per_step": world * sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg)),
               "d2h_bytes_per_step": world * hy.numel() * hy.element_size(),
               "api": ("speed3r_b200.HostPipeline (head group by head group: K, V, then queries by chunk; copies overlapped with kernels)"
                       if pipe is not None else "speed3r_b200.seq_parallel.sparse_attention_partitioned on this rank's shard")}

    # The whole module (qkv/gate/proj GEMMs + prologue + the op) at the same sequence length, forward, no
    # gradients: once with the one-pass prologue kernel, once with the separate PyTorch steps around the op.
    module = None
    if world == 1 and not bwd and args.module:
        import speed3r_b200
        del q, k, v, gate
        if not args.no_e2e:
            del pipe, hq, hk, hv, hg, hy
        torch.cuda.empty_cache()
        dim = H * D
        mod = speed3r_b200.SparseFlashAttentionRope(dim, num_heads=H, qkv_bias=True, proj_bias=True, qk_norm=True,
                                                    rope=speed3r_b200.RoPE2D(100.0)).to(dev).eval()
        gm = torch.Generator(device=dev).manual_seed(7)
        x = torch.randn(1, T, dim, device=dev, generator=gm).bfloat16()
        side = int(math.sqrt(TOK_PER_VIEW))            # token grid of one view, for plausible (y,x) positions
        tok = torch.arange(T, device=dev) % TOK_PER_VIEW
        xpos = torch.stack((tok // (TOK_PER_VIEW // side), tok % (TOK_PER_VIEW // side)), -1)[None].contiguous()

        def time_module(fused):
            mod._can_fuse_prologue = (lambda *a, **k_: False) if not fused else type(mod)._can_fuse_prologue.__get__(mod)
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                mod(x, xpos=xpos)
                torch.cuda.synchronize()
                a, b_ = ev(), ev()
                a.record()
                for _ in range(2):
                    mod(x, xpos=xpos)
                b_.record()
                torch.cuda.synchronize()
            return a.elapsed_time(b_) / 2
        module = {"tokens": T, "dim": dim, "fused_prologue_ms": time_module(True), "separate_steps_ms": time_module(False)}
        del mod, x

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cstep, cfl, sample, cores = cpu_sample(args.views)
        cstep()
        c0 = time.perf_counter()
        nrep = 2
        for _ in range(nrep):
            cstep()
        cdt = (time.perf_counter() - c0) / nrep
        cpu = {"value": cfl / cdt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample,
               "s_per_sample": cdt}

    if rank == 0:
        line = dict(metric="sparse_attn_layer_effective_tflops", value=value, unit="TFLOP/s", n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="strong",
                    vs_baseline=None, dtype="bf16", data="synthetic", config=workload_config(args),
                    views_per_s=args.views / (ms * 1e-3), clocks=clocks, e2e=e2e,
                    # own kernels per step and rank: 3 pool + compression attention + selection/merge
                    # (+ with the backward: merge bwd, 4 CSR, 2 selection bwd, delta + 2 compression bwd, 3 pool bwd)
                    gpu_launches=args.steps * world * (5 if not bwd else 5 + 1 + 4 + 2 + 3 + 3),
                    roofline=roof, kernels=kern, cpu_baseline=cpu)
        if module is not None:
            line["module"] = module
        if parity is not None:
            line["parity"] = parity
        if tri is not None:
            line["triton_baseline"] = tri
            if "total_ms" in tri and kern is not None:
                line["triton_baseline"]["speedup_of_ours"] = tri["total_ms"] / (kern["cmp_attn_topk_ms"] + kern["sel_attn_merge_ms"])
        if dense is not None:
            line["dense_baseline"] = dense
            if "ms" in dense:
                line["dense_baseline"]["fraction_of_dense_time"] = ms / dense["ms"]
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
