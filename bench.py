"""Benchmark of the optimizer-step hot path: AdamW bf16 + Kahan on Llama-3-8B parameter shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl optimi_b200|reference] [--workload NAME]

One "step" is one optimizer step over the whole parameter list (synthetic, seeded; no dataset).
Prints ONE JSON line (rank 0).  For N > 1 launch under torchrun; the optimizer states are sharded
ZeRO-1 style (optimi_b200.zero.ShardedOptimizer): each rank steps 1/N of the elements and the updated
bf16 parameters reach the other ranks either inside the step kernel (peer stores over NVLink,
--exchange push, the default where available) or by an NCCL all-gather after it (--exchange nccl).
Total work is fixed, so scaling is "strong".

Keys beyond the driver's contract:
  roofline      dominant kernel against the HBM copy peak (MEASURED_PEAKS.json, else the fallback)
  cpu_baseline  the reference's own foreach path on this host's cores (or the C oracle port when the
                reference package is not present), on a bounded sample of the same workload
  e2e           the same metric through the public API with gradients arriving from pinned host
                memory every step and a small device-to-host read of the result
  step_ms / gather_ms   device time of the local step and of the all-gather (N > 1)
  exchange_check        N > 1: after the warm-up steps every rank checksums its whole parameter buffers and the ranks
                        compare; the run exits non-zero when they differ
  local_step_ms         N > 1: the rank's step alone (no exchange), i.e. the per-rank step time
  reference_gpu         N = 1: the reference's own CUDA back ends (foreach, Triton) and this build on the 1.1 B list
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "AdamW bf16-Kahan step: Gparams/s & HBM GB/s vs 8 TB/s, 8B shapes, 1/2/4/8 GPU"
UNIT = "Gparams/s"
BYTES_PER_PARAM = 18  # read p,g,m,v,k (10 B) + write p,m,v,k (8 B), bf16 + Kahan
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per parameter of the bf16+Kahan kernels, from ncu captures of a
# 336 M-parameter list (StableAdamW: both passes together); traffic is proportional to the parameter count, so a
# step's traffic is this figure times its elements
NCU_DRAM_BYTES_PER_PARAM = {"adamw": 17.83, "adam": 17.83, "lion": 13.83, "adan": 25.84, "stableadamw": 21.70}

HYPER = dict(lr=3e-4, betas=(0.9, 0.99), weight_decay=1e-5, eps=1e-6, decouple_lr=True)

# --optimizer: class name, constructor keywords (BASELINE configs 3 and 4), algorithmic bytes per parameter in
# bf16 + Kahan (streams read + written, 2 B each), kernel name for the roofline object
OPTIMIZERS = {
    "adamw": ("AdamW", HYPER, 18, "mta_kernel<bf16, AdamOp<kahan,update>>"),
    "adam": ("Adam", dict(lr=3e-4, betas=(0.9, 0.99), eps=1e-6), 18, "mta_kernel<bf16, AdamOp<kahan,update>>"),
    "lion": ("Lion", dict(lr=1e-4, betas=(0.9, 0.99)), 14, "mta_kernel<bf16, LionOp<kahan,update>>"),
    "sgd": ("SGD", dict(lr=1e-2, momentum=0.9), 14, "mta_kernel<bf16, SgdOp<kahan,update>>"),
    "stableadamw": ("StableAdamW", dict(lr=3e-4), 22, "tile_sum_kernel<bf16, StableMomentsOp> + mta_kernel<bf16, StableUpdateOp<kahan>>"),
    "adan": ("Adan", dict(lr=3e-4, betas=(0.98, 0.92, 0.99), kahan_sum=True), 26, "mta_kernel<bf16, AdanOp<kahan,update>>"),
    "radam": ("RAdam", dict(lr=3e-4), 18, "mta_kernel<bf16, RangerOp<kahan,update>>"),
    # Lookahead (k=6) reads and writes the slow weights on every 6th step: 18 + 4/6 bytes on average
    "ranger": ("Ranger", dict(lr=3e-4, k=6, alpha=0.5), 18 + 4 / 6, "mta_kernel<bf16, RangerOp<kahan,update>>"),
}


def metric_name(optimizer: str) -> str:
    if optimizer == "adamw":
        return METRIC
    return f"{OPTIMIZERS[optimizer][0]} bf16-Kahan step: Gparams/s & HBM GB/s vs 8 TB/s, 1/2/4/8 GPU"


def llama_shapes(hidden, layers, ffn, q_heads, kv_heads, head_dim, vocab):
    """Parameter shapes of a Llama-style decoder in Hugging Face order (untied output head)."""
    shapes = [(vocab, hidden)]
    for _ in range(layers):
        shapes += [
            (q_heads * head_dim, hidden), (kv_heads * head_dim, hidden), (kv_heads * head_dim, hidden),
            (hidden, q_heads * head_dim), (ffn, hidden), (ffn, hidden), (hidden, ffn), (hidden,), (hidden,),
        ]  # fmt: skip
    shapes += [(hidden,), (vocab, hidden)]
    return shapes


WORKLOADS = {
    "llama3-8b": lambda: llama_shapes(4096, 32, 14336, 32, 8, 128, 128256),
    "llama-1.1b": lambda: llama_shapes(2048, 22, 5632, 32, 4, 64, 32000),
    "llama-3b": lambda: llama_shapes(3072, 28, 8192, 24, 8, 128, 128256),
    "llama-0.3b": lambda: llama_shapes(1024, 24, 2816, 16, 4, 64, 32000),  # small case for profiler captures
    "tiny": lambda: llama_shapes(256, 2, 688, 4, 2, 64, 1024),
}


def numel(shape):
    return math.prod(shape)


def make_config(workload: str, n_gpus: int, exchange: str = "auto", optimizer: str = "adamw") -> dict:
    """The `config` object of the JSON line; identical for both arms of one (workload, N)."""
    shapes = WORKLOADS[workload]()
    n_params = sum(numel(s) for s in shapes)
    sample = cpu_sample_shapes(workload)
    return {
        # the same text in both arms; it also says what the CPU reference arm, which cannot step the whole list within
        # minutes, times per step (its ms_per_step is that sample's, its value the sample's parameters per second)
        "workload": f"{OPTIMIZERS[optimizer][0]} bf16+Kahan, {workload} parameter shapes ({n_params} params, {len(shapes)} tensors); "
                    f"the CPU reference arm times a bounded sample per step: the first decoder layer, {len(sample)} tensors, "
                    f"{sum(numel(x) for x in sample)} params",
        "optimizer": OPTIMIZERS[optimizer][0], "hyper": {k: (list(v) if isinstance(v, tuple) else v) for k, v in OPTIMIZERS[optimizer][1].items()},
        "sharding": "none" if n_gpus == 1 else f"ZeRO-1 over {n_gpus} ranks, exchange={exchange} "
                    "(push: step kernel stores updated params into the peers over NVLink; nccl: all-gather after the step)",
        "l2": "inputs larger than L2, no flush between steps: %.1f GB streamed per rank per step" % (OPTIMIZERS[optimizer][2] * n_params / n_gpus / 1e9),
    }  # fmt: skip


def make_params(shapes, device, dtype, seed=0):
    """2-D weights ~N(0, 0.02^2), 1-D (norm) weights = 1."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = []
    for s in shapes:
        if len(s) == 1:
            out.append(torch.ones(s, device=device, dtype=dtype))
        else:
            out.append(torch.randn(s, device=device, dtype=torch.float32, generator=g).mul_(0.02).to(dtype))
    return out


def grad_scales(n, seed=0):
    """Per-tensor gradient scale ~LogNormal(ln 1e-3, 1)."""
    g = torch.Generator().manual_seed(seed)
    return torch.exp(torch.randn(n, generator=g) + math.log(1e-3)).tolist()


def fill_grad(t, scale, gen):
    """N(0,1) * scale into `t`, chunked so the fp32 temporary stays small."""
    flat = t.view(-1)
    step = 1 << 26
    for a in range(0, flat.numel(), step):
        b = min(a + step, flat.numel())
        flat[a:b] = torch.randn(b - a, device=t.device, dtype=torch.float32, generator=gen).mul_(scale).to(t.dtype)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = None
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: rank 0 prints one JSON line
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's foreach path (or the oracle port) on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_sample_shapes(workload):
    """A bounded sample of the workload: the tensors of its first decoder layer."""
    shapes = WORKLOADS[workload]()
    return shapes[1:10]


def time_cpu_reference(workload, steps, warmup, budget_s=25.0, optimizer="adamw"):
    """Returns (Gparams/s, kind, cores, sample description).  One step = one optimizer step over the
    sample, AdamW bf16 + Kahan with the benchmark's hyper-parameters, all host threads."""
    shapes = cpu_sample_shapes(workload)
    n = sum(numel(s) for s in shapes)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    params = [p.requires_grad_(True) for p in make_params(shapes, "cpu", torch.bfloat16, seed=1)]
    scales = grad_scales(len(shapes), seed=1)
    gen = torch.Generator().manual_seed(1001)
    grads = [torch.randn(s, generator=gen).mul_(sc).to(torch.bfloat16) for s, sc in zip(shapes, scales)]
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    kind = "port"
    if os.path.isdir(os.path.join(ref_dir, "optimi")):
        sys.path.insert(0, ref_dir)
        try:
            import warnings

            import optimi  # the unmodified reference package

            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                opt = getattr(optimi, OPTIMIZERS[optimizer][0])(params, foreach=True, triton=False, **OPTIMIZERS[optimizer][1])
            kind = "reference"

            def one_step():
                for p, g in zip(params, grads):
                    p.grad = g.clone()  # the foreach path clobbers gradients
                t0 = time.perf_counter()
                opt.step()
                return time.perf_counter() - t0
        except Exception:
            kind = "port"
    if kind == "port":
        from oracle.port import OracleOptimizer

        opt = OracleOptimizer(optimizer, [p.detach() for p in params], **OPTIMIZERS[optimizer][1])

        def one_step():
            gs = [g.clone() for g in grads]
            t0 = time.perf_counter()
            opt.step(gs)
            return time.perf_counter() - t0

    for _ in range(warmup):
        one_step()
    times, t_start = [], time.perf_counter()
    for _ in range(steps):
        times.append(one_step())
        if time.perf_counter() - t_start > budget_s:
            break
    sec = statistics.median(times)
    sample = f"first decoder layer of {workload}: {len(shapes)} tensors, {n} params, {len(times)} timed steps (median), grads re-cloned untimed"
    return n / sec / 1e9, kind, cores, sample, sec * 1e3, len(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, kind, cores, sample, ms, done = time_cpu_reference(args.workload, args.steps, args.warmup, budget_s=150.0, optimizer=args.optimizer)
    config = make_config(args.workload, args.gpus, args.exchange, args.optimizer)
    line = {
        "impl": "reference", "metric": metric_name(args.optimizer), "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": done,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# the optimi_b200 arm
# ------------------------------------------------------------------------------------------------
def make_reduce_probe(sharded, params, opt_cls, opt_kw, world):
    """--reduce-grads: an unsharded twin of ONE tensor that straddles a shard boundary, stepped on the mean of all
    ranks' gradients (fp32 sum in rank order, times 1/world, one rounding: the fused kernel's arithmetic) beside
    the sharded warm-up steps; the two must stay bit-identical."""
    import torch.distributed as dist

    b = sharded.buckets[0]
    layout = b["layout"]
    cut = layout.bounds[1]
    pick = next((i for i, (off, n) in enumerate(zip(layout.offsets, layout.numels)) if off < cut < off + n), 0)
    p = b["params"][pick]
    gathered = [torch.empty_like(p.grad) for _ in range(world)]
    dist.all_gather(gathered, p.grad.contiguous())
    acc = gathered[0].float()
    for g in gathered[1:]:
        acc += g.float()
    twin = p.detach().clone().requires_grad_(True)
    twin.grad = (acc * (1.0 / world)).to(p.dtype)
    del gathered, acc
    return {"opt": opt_cls([twin], **opt_kw), "twin": twin, "sharded_tensor": p,
            "describe": f"tensor {pick} {tuple(p.shape)}, cut by the boundary between ranks 0 and 1"}  # fmt: skip


def measure_peer_copy_gbs(nbytes=1 << 30, repeats=5):
    """GB/s of a plain device-to-device copy from GPU 0 to GPU 1 (two ordinary allocations, one per device, the
    runtime's peer copy; best of `repeats`): the per-direction NVLink rate the exchange is held against."""
    if torch.cuda.device_count() < 2:
        return None
    try:
        src = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0")
        dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda:1")
        dst.copy_(src)
        torch.cuda.synchronize("cuda:0")
        torch.cuda.synchronize("cuda:1")
        best = float("inf")
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.device(0):
                e0.record()
                dst.copy_(src, non_blocking=True)
                e1.record()
                e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        del src, dst
        return nbytes / (best * 1e-3) / 1e9
    except RuntimeError:
        return None


def time_reference_gpu(device, steps=10):
    """The reference's own CUDA back ends and this build on ONE list on this GPU (the 1.1 B Llama-style list, AdamW
    bf16 + Kahan, decouple_lr): `optimi.AdamW(foreach=True)` and `(triton=True)` from the unmodified reference package
    beside `optimi_b200.AdamW`, CUDA events around `steps` steps each after 3 warm-up steps."""
    import warnings

    import optimi_b200

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        return {"kind": "unavailable", "why": "reference package not present beside the repository"}
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import optimi

    workload = "llama-1.1b"
    shapes = WORKLOADS[workload]()
    n = sum(numel(s) for s in shapes)
    scales = grad_scales(len(shapes), seed=0)
    out = {"workload": f"AdamW bf16+Kahan, {workload} parameter shapes ({n} params, {len(shapes)} tensors)", "steps": steps, "unit": "ms per step"}

    def one(make, clobbers):
        params = [p.requires_grad_(True) for p in make_params(shapes, device, torch.bfloat16, seed=0)]
        gen = torch.Generator(device=device).manual_seed(5)
        grads = []
        for p, sc in zip(params, scales):
            g = torch.empty_like(p)
            fill_grad(g, sc, gen)
            grads.append(g)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            opt = make(params)

        def step():
            for p, g in zip(params, grads):
                p.grad = g.clone() if clobbers else g  # the reference's foreach path uses its gradients as scratch
            opt.step()

        for _ in range(3):
            step()
        torch.cuda.synchronize(device)
        total = 0.0
        for _ in range(steps):
            for p, g in zip(params, grads):
                p.grad = g.clone() if clobbers else g
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            opt.step()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        del opt, params, grads
        torch.cuda.empty_cache()
        return total / steps

    out["optimi_b200"] = one(lambda ps: optimi_b200.AdamW(ps, **HYPER), False)
    for key, kw, clobbers in (("reference_foreach", dict(foreach=True, triton=False), True), ("reference_triton", dict(foreach=False, triton=True), False)):
        try:
            out[key] = one(lambda ps: optimi.AdamW(ps, **HYPER, **kw), clobbers)
        except Exception as exc:  # e.g. Triton cannot compile on this machine
            out[key] = None
            out[key + "_unavailable"] = f"{type(exc).__name__}: {exc}"[:200]
    out["kind"] = "measured"
    return out


def run_b200_arm(args):
    import optimi_b200
    from optimi_b200 import _lib
    from optimi_b200.zero import ShardedOptimizer

    world, rank, local = dist_setup(args.gpus)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    # fp16 and fp32 are secondary figures; the metric is quoted on bf16
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    shapes = WORKLOADS[args.workload]()
    n_params = sum(numel(s) for s in shapes)

    cls_name, opt_kw, bytes_per_param, kernel_name = OPTIMIZERS[args.optimizer]
    if args.dtype == "fp32":
        # float32 has no Kahan buffer: one 4-byte stream fewer in each direction than the 2-byte count, all streams 4 bytes
        bytes_per_param = (bytes_per_param - 4) * 2
        opt_kw = {k: v for k, v in opt_kw.items() if k != "kahan_sum"}
        kernel_name = kernel_name.replace("bf16", "f32").replace("kahan,", "").replace("<kahan>", "")
    opt_cls = getattr(optimi_b200, cls_name)
    params = [p.requires_grad_(True) for p in make_params(shapes, device, dtype, seed=0)]
    if world == 1:
        opt = opt_cls(params, **opt_kw)
        step_targets = params
        sharded = None
    else:
        # the list goes in as 8 x N consecutive parameter groups (same options), so that the end-to-end path can step a
        # rank's range in about eight pieces as its gradients land; the device-timed steps run all groups back to back
        n_groups, target, acc, groups = 8 * world, n_params / (8 * world), 0, []
        for p in params:
            gi = min(n_groups - 1, int(acc / target))
            while len(groups) <= gi:
                groups.append({"params": []})
            groups[gi]["params"].append(p)
            acc += p.numel()
        groups = [g for g in groups if g["params"]]
        sharded = ShardedOptimizer(opt_cls, groups, exchange=args.exchange, reduce_grads=args.reduce_grads, **opt_kw)
        opt = sharded
        step_targets = sharded.shard_params
    n_local = sum(t.numel() for t in step_targets)

    # gradients resident in HBM for the `value` arm: one tensor per stepped tensor
    scales = grad_scales(len(shapes), seed=0)
    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    if sharded is None:
        piece_scale = scales
    else:
        piece_scale = [scales[i] for b in sharded.buckets for (i, _, _) in b["pieces"]]
    dev_grads = []
    if args.reduce_grads:
        # data-parallel form: every rank holds FULL gradients (its own micro-batch's) in the shared buffer and the
        # step kernel averages them across ranks as it goes
        sharded.attach_grads()
        for p, sc in zip(params, scales):
            fill_grad(p.grad, sc, gen)
    else:
        for t, sc in zip(step_targets, piece_scale):
            g = torch.empty_like(t)
            fill_grad(g, sc, gen)
            dev_grads.append(g)

    def step_resident():
        if sharded is None:
            opt.step()
        elif args.reduce_grads:
            sharded.step()
        else:
            sharded.step(dev_grads)

    for t, g in zip(step_targets, dev_grads):
        t.grad = g

    # ---- kernel-resident timing ---------------------------------------------------------------
    probe = make_reduce_probe(sharded, params, opt_cls, opt_kw, world) if (sharded is not None and args.reduce_grads) else None
    for _ in range(max(args.warmup, 3)):
        step_resident()
        if probe is not None:
            probe["opt"].step()
    barrier(world)
    # outside the timed region: do all ranks hold the same bits after the sharded warm-up steps?
    exchange_check = None
    if sharded is not None:
        exchange_check = sharded.check_replicas()
        if probe is not None:
            exchange_check["matches_unsharded_on_mean_gradient"] = bool(torch.equal(probe["sharded_tensor"].detach(), probe["twin"].detach()))
            exchange_check["probe_tensor"] = probe["describe"]
            del probe
        ok = exchange_check["ranks_identical"] and exchange_check.get("matches_unsharded_on_mean_gradient", True)
        if not ok:
            if rank == 0:
                print(json.dumps({"error": "sharded step left the ranks with different parameters", "exchange_check": exchange_check}))
            raise SystemExit(3)
    stream = torch.cuda.current_stream(device)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = _lib.LIB.optimi_b200_launch_count()
    with ClockSampler(local) as clocks:
        barrier(world)
        torch.cuda.profiler.start()  # lets a profiler started with --profile-from-start off see only the timed region
        t_wall = time.perf_counter()
        for k in range(args.steps):
            ev[k][0].record(stream)
            if sharded is None:
                opt.step()
                ev[k][1].record(stream)
            else:
                sharded.step_local(None if args.reduce_grads else dev_grads)
                ev[k][1].record(stream)
                sharded.gather_params()
            ev[k][2].record(stream)
        barrier(world)
        t_wall = time.perf_counter() - t_wall
        torch.cuda.profiler.stop()
    launches = _lib.LIB.optimi_b200_launch_count() - launches0
    total_ms = ev[0][0].elapsed_time(ev[-1][2])
    step_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    gather_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    # spread of the whole step (local step + exchange) over the timed steps of this rank, as the reference's own
    # benchmark reports it (mean / median / p90, examples/benchmark.py:373-381)
    per_step = sorted(e[0].elapsed_time(e[2]) for e in ev)
    spread = {"mean": sum(per_step) / len(per_step), "median": per_step[len(per_step) // 2],
              "p90": per_step[min(len(per_step) - 1, int(0.9 * len(per_step)))], "min": per_step[0], "max": per_step[-1]}  # fmt: skip
    total_ms = max_over_ranks(total_ms, world, device)
    step_ms_max = max_over_ranks(step_ms, world, device)
    gather_ms_max = max_over_ranks(gather_ms, world, device)
    ms_per_step = total_ms / args.steps
    value = n_params / (ms_per_step * 1e-3) / 1e9

    # ---- N > 1: the rank's step alone, without the exchange (the per-rank step time) ----------------
    local_step_ms = None
    if sharded is not None and not args.reduce_grads:
        k_local = max(3, min(args.steps, 10))
        sharded.step_local(dev_grads, exchange=False)
        barrier(world)
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record(stream)
        for _ in range(k_local):
            sharded.step_local(dev_grads, exchange=False)
        l1.record(stream)
        barrier(world)
        local_step_ms = max_over_ranks(l0.elapsed_time(l1) / k_local, world, device)
        sharded.gather_params(force=True)  # the ranks' copies diverged during the local-only steps: bring them together again
        barrier(world)

    # ---- end to end: gradients from pinned host memory, result read back -----------------------
    if args.reduce_grads:
        dev_grads = [p.grad for p in params]  # end to end: each rank's full gradients arrive from the host
    host_grads = [torch.empty(g.shape, dtype=g.dtype, pin_memory=True) for g in dev_grads]
    for h, g in zip(host_grads, dev_grads):
        h.copy_(g)
    result_src = params[-2]  # the final norm weight: a small tensor every rank holds after the exchange
    result_host = torch.empty(result_src.shape, dtype=result_src.dtype, pin_memory=True)
    h2d_bytes = sum(h.numel() * h.element_size() for h in host_grads)
    d2h_bytes = result_host.numel() * result_host.element_size()

    e2e_overlap = None
    if sharded is None:
        # one GPU: the gradients arrive in chunks on a copy stream and every chunk is stepped as soon as it has
        # landed (OptimiOptimizer.step_groups over one param group per chunk), so that only the last chunk's step
        # is not hidden behind the PCIe transfer.  A fresh optimizer over the same parameters, grouped by chunk.
        n_chunks = 16
        del opt
        torch.cuda.empty_cache()
        order, acc, chunk_of, target = list(range(len(params))), 0, [], n_params / n_chunks
        for i in order:
            chunk_of.append(min(n_chunks - 1, int(acc / target)))
            acc += params[i].numel()
        chunks = [[i for i in order if chunk_of[i] == c] for c in range(n_chunks)]
        chunks = [c for c in chunks if c]
        opt = opt_cls([{"params": [params[i] for i in c]} for c in chunks], **opt_kw)
        copy_stream = torch.cuda.Stream(device)
        landed = [torch.cuda.Event() for _ in chunks]
        e2e_overlap = {"chunks": len(chunks), "how": "gradient chunks copied on a side stream, each stepped (step_groups) when its copy has landed"}

        def step_e2e():
            main = torch.cuda.current_stream(device)
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                for ci, c in enumerate(chunks):
                    for i in c:
                        dev_grads[i].copy_(host_grads[i], non_blocking=True)
                    landed[ci].record(copy_stream)
            for ci in range(len(chunks)):
                main.wait_event(landed[ci])
                opt.step_groups([ci])
            result_host.copy_(result_src.detach(), non_blocking=True)
            main.synchronize()

    elif not args.reduce_grads:
        # N > 1: the same, over this rank's pieces of each parameter group (ShardedOptimizer.begin_step / step_groups /
        # end_step); a rank's range touches about eight of the 8 x N groups
        index_of = {id(t): i for i, t in enumerate(step_targets)}
        pieces_of_group = [[index_of[id(sp)] for sp in g["params"]] for g in sharded.inner.param_groups]
        mine = [gi for gi, idx in enumerate(pieces_of_group) if idx]
        copy_stream = torch.cuda.Stream(device)
        landed = {gi: torch.cuda.Event() for gi in mine}
        e2e_overlap = {"chunks": len(mine), "how": "this rank's gradient pieces copied group by group on a side stream, each group stepped "
                       "(and pushed) when its copy has landed"}  # fmt: skip

        def step_e2e():
            main = torch.cuda.current_stream(device)
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                for gi in mine:
                    for i in pieces_of_group[gi]:
                        dev_grads[i].copy_(host_grads[i], non_blocking=True)
                    landed[gi].record(copy_stream)
            sharded.begin_step(dev_grads)
            for gi in range(len(pieces_of_group)):
                if gi in landed:
                    main.wait_event(landed[gi])
                sharded.step_groups([gi])  # every group on every rank: the step counters of all groups advance together
            sharded.end_step()
            result_host.copy_(result_src.detach(), non_blocking=True)
            main.synchronize()

    else:

        def step_e2e():
            for h, g in zip(host_grads, dev_grads):
                g.copy_(h, non_blocking=True)
            step_resident()
            result_host.copy_(result_src.detach(), non_blocking=True)
            torch.cuda.current_stream(device).synchronize()

    e2e_steps = max(2, min(args.steps, 5))
    step_e2e()
    barrier(world)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    barrier(world)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device) / e2e_steps
    e2e_value = n_params / e2e_s / 1e9

    if rank != 0:
        return

    # ---- roofline of the dominant kernel (the step kernel) -------------------------------------
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as fh:
            peak, peak_kind = float(json.load(fh)["hbm_gbs"]), "measured"
    else:
        peak, peak_kind = FALLBACK_HBM_GBS, "fallback"
    kernel_launches_per_step = max(1, launches // args.steps)
    # the kernel against HBM: at N > 1 with the push exchange `step_ms` is NVLink-bound (it contains the exchange), so the
    # roofline of the step kernel is taken from the local-only steps timed above
    kernel_ms = local_step_ms if local_step_ms is not None else step_ms_max
    achieved = bytes_per_param * n_local / (kernel_ms * 1e-3) / 1e9
    ncu_bpp = NCU_DRAM_BYTES_PER_PARAM.get(args.optimizer) if args.dtype == "bf16" else None  # the captures are of the bf16 kernels
    traffic = ncu_bpp * n_local / kernel_launches_per_step if ncu_bpp is not None else None
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
        "traffic_note": (f"bytes per launch: ncu dram read+write of a 336 M-param capture ({ncu_bpp} B/param per step) scaled by "
                         "elements per launch" if ncu_bpp is not None else "no ncu capture of this kernel"),
        "peak_kind": f"of {peak_kind}", "frac_of_8TBs": achieved / 8000.0, "kernel": kernel_name,
        "algorithmic_bytes_per_launch": bytes_per_param * n_local / kernel_launches_per_step,
        "algorithmic_bytes_per_param": bytes_per_param,
        "launches_per_step": kernel_launches_per_step, "kernel_ms": kernel_ms,
        "timed_as": "local-only steps (no exchange) after the timed region" if local_step_ms is not None else "the timed steps",
    }  # fmt: skip

    nvlink = None
    if sharded is not None:
        # what must cross NVLink per rank and step, against a peer copy measured in this very run (GPU 0 -> GPU 1,
        # 1 GiB, best of 5); the nominal 900 GB/s per direction stands in when it cannot be measured
        link_gbs = measure_peer_copy_gbs()
        link_kind = "measured in this run" if link_gbs is not None else "nominal"
        link_gbs = link_gbs or 900.0
        pushed = 2.0 * n_local * (world - 1)  # bytes this rank's updated parameters occupy on its peers
        # with --reduce-grads the same link direction also carries the responses to the peers' gradient reads
        pulled = pushed if args.reduce_grads else 0.0
        exchange_ms = step_ms_max if sharded.exchange == "push" else gather_ms_max
        nvlink = {"achieved": (pushed + pulled) / (exchange_ms * 1e-3) / 1e9, "peak": link_gbs, "peak_kind": link_kind,
                  "unit": "GB/s per direction per GPU", "frac": (pushed + pulled) / (exchange_ms * 1e-3) / 1e9 / link_gbs,
                  "bytes_pushed_per_rank_per_step": pushed, "bytes_pulled_per_rank_per_step": pulled,
                  "exchange_bound_ms": (pushed + pulled) / (link_gbs * 1e9) * 1e3,
                  "timed_over": "the fused step kernel" if sharded.exchange == "push" else "the all-gather"}

    reference_gpu = None
    if world == 1 and not args.no_reference_gpu:
        del opt, host_grads, dev_grads, params, step_targets
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        reference_gpu = time_reference_gpu(device)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        v, kind, cores, sample, _, _ = time_cpu_reference(args.workload, 12, 2, budget_s=20.0, optimizer=args.optimizer)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample}

    # per-rank step time against the one-GPU step: t1 / (N * tN), t1 taken from a one-GPU run of the same workload on this
    # machine if one left its record (the scaling series runs N = 1 first), else from this run's own HBM rate
    t1_path = os.path.join("/tmp", f"optimi_b200_bench_t1_{args.workload}_{args.optimizer}.json")
    local_eff = None
    if world == 1:
        try:
            with open(t1_path, "w") as fh:
                json.dump({"step_ms": step_ms_max, "when": time.time()}, fh)
        except OSError:
            pass
    elif local_step_ms is not None:
        try:
            with open(t1_path) as fh:
                rec = json.load(fh)
            if time.time() - rec["when"] < 6 * 3600:
                local_eff = {"value": rec["step_ms"] / (world * local_step_ms), "t1_ms": rec["step_ms"], "t1_from": "one-GPU run on this machine"}
        except (OSError, ValueError, KeyError):
            pass
    bound = None
    if sharded is not None:
        bound = ("nvlink: the step kernel also stores every updated parameter into the peers" if sharded.exchange == "push"
                 else "nvlink: the all-gather after the step")

    line = {
        "metric": metric_name(args.optimizer), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": args.dtype,
        "data": "synthetic",
        "config": make_config(args.workload, world, args.exchange, args.optimizer),
        "exchange": None if sharded is None else sharded.exchange, "reduce_grads": bool(args.reduce_grads),
        "hbm_gbs": achieved, "step_ms": step_ms_max, "gather_ms": gather_ms_max, "wall_ms_per_step": t_wall * 1e3 / args.steps,
        "step_ms_spread_rank0": spread,
        "exchange_check": exchange_check, "local_step_ms": local_step_ms, "local_step_efficiency": local_eff, "bound": bound,
        "roofline": roofline, "nvlink": nvlink, "cpu_baseline": cpu, "reference_gpu": reference_gpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": e2e_s * 1e3, "steps": e2e_steps, "overlap": e2e_overlap},
        "gpu_launches": int(launches), "clocks": clocks.result, "library": os.path.relpath(_lib.LIB_PATH, ROOT),
    }  # fmt: skip
    if args.dtype != "bf16":  # say what was stepped where the line names the workload
        label = "fp16+Kahan" if args.dtype == "fp16" else "fp32 (no Kahan buffer)"
        line["metric"] = line["metric"].replace("bf16-Kahan", label)
        line["config"]["workload"] = line["config"]["workload"].replace("bf16+Kahan", label)
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# secondary workload: gradient release + optimizer accumulation inside a real backward pass
# ------------------------------------------------------------------------------------------------
def run_gradient_release(args):
    """BASELINE config 5: 24-layer GPT-style decoder (d_model 1024, 16 heads, FFN 4096, vocab 50304, bf16, 388
    parameter tensors), random token ids at batch 8 x seq 1024, AdamW + Kahan stepping from backward hooks with
    4-step optimizer accumulation.  Reports device milliseconds per micro-step (forward + backward + released
    steps) for: no optimizer at all, optimi_b200 hooks on the backward stream, optimi_b200 hooks on a side stream,
    and the reference's hooks with its Triton and ATen back ends when the reference package is present."""
    import warnings

    import torch.nn as nn
    import torch.nn.functional as Fn

    import optimi_b200

    warnings.simplefilter("ignore")
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    optimi = None
    if os.path.isdir(os.path.join(ref_dir, "optimi")):
        sys.path.insert(0, ref_dir)
        import optimi

    class Block(nn.Module):
        def __init__(self, d, h, f):
            super().__init__()
            self.h = h
            self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.q, self.k, self.v, self.o = nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d)
            self.fc, self.proj = nn.Linear(d, f), nn.Linear(f, d)

        def forward(self, x):
            B, S, D = x.shape
            y = self.ln1(x)
            q, k, v = (m(y).view(B, S, self.h, D // self.h).transpose(1, 2) for m in (self.q, self.k, self.v))
            x = x + self.o(Fn.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, D))
            return x + self.proj(Fn.gelu(self.fc(self.ln2(x))))

    class GPT(nn.Module):
        def __init__(self, layers=24, d=1024, h=16, f=4096, vocab=50304, ctx=1024):
            super().__init__()
            self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(ctx, d)
            self.blocks = nn.ModuleList([Block(d, h, f) for _ in range(layers)])
            self.ln_f = nn.LayerNorm(d)

        def forward(self, idx):
            x = self.wte(idx) + self.wpe(torch.arange(idx.shape[1], device=idx.device))
            for b in self.blocks:
                x = b(x)
            return self.ln_f(x) @ self.wte.weight.t()

    def run(mode):
        torch.manual_seed(0)
        model = GPT().to("cuda", torch.bfloat16)
        params = list(model.parameters())
        kw = dict(lr=3e-4, weight_decay=1e-2)
        opt = None
        if mode.startswith("optimi_b200"):
            opt = optimi_b200.AdamW(params, gradient_release=True, **kw)
            optimi_b200.prepare_for_gradient_release(model, opt, side_stream=mode.endswith("side_stream"))
        elif mode.startswith("reference"):
            opt = optimi.AdamW(params, gradient_release=True, triton=mode.endswith("triton"), foreach=False, **kw)
            optimi.prepare_for_gradient_release(model, opt)
        gen = torch.Generator(device="cuda").manual_seed(1)

        def micro(i):
            if opt is not None:
                opt.optimizer_accumulation = i % 4 != 3
            idx = torch.randint(0, 50304, (8, 1024), device="cuda", generator=gen)
            Fn.cross_entropy(model(idx).float().view(-1, 50304), idx.view(-1)).backward()
            if opt is None and i % 4 == 3:
                for p in params:
                    p.grad = None

        for i in range(8):
            micro(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = optimi_b200._lib.LIB.optimi_b200_launch_count()
        e0.record()
        for i in range(args.steps):
            micro(i)
        e1.record()
        torch.cuda.synchronize()
        return {"ms_per_micro_step": e0.elapsed_time(e1) / args.steps, "n_tensors": len(params),
                "n_params": sum(p.numel() for p in params), "peak_gb": torch.cuda.max_memory_allocated() / 1e9,
                "gpu_launches": optimi_b200._lib.LIB.optimi_b200_launch_count() - launches0}  # fmt: skip

    modes = ["no_optimizer", "optimi_b200_backward_stream", "optimi_b200_side_stream"] + (["reference_triton", "reference_aten"] if optimi else [])
    res = {}
    for m in modes:
        torch.cuda.reset_peak_memory_stats()
        res[m] = run(m)
        import gc

        gc.collect()  # the hooks keep model <-> optimizer cycles alive until collected
        torch.cuda.empty_cache()
    base = res["no_optimizer"]["ms_per_micro_step"]
    line = {
        "metric": "gradient release + 4-step optimizer accumulation, AdamW bf16+Kahan: device ms per micro-step (fwd+bwd+released steps)",
        "value": res["optimi_b200_side_stream"]["ms_per_micro_step"],  # the default: released steps on a side stream "unit": "ms", "higher_is_better": False, "n_gpus": 1, "steps": args.steps,
        "config": {"workload": "24-layer GPT-style decoder, d_model 1024, 16 heads, FFN 4096, vocab 50304, bf16, batch 8 x seq 1024"},
        "data": "synthetic", "dtype": "bf16", "results": res,
        "optimizer_overhead_ms": {k: v["ms_per_micro_step"] - base for k, v in res.items() if k != "no_optimizer"},
    }  # fmt: skip
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="optimi_b200", choices=["optimi_b200", "reference"])
    ap.add_argument("--workload", default="llama3-8b", choices=sorted(WORKLOADS) + ["gpt-gradient-release"])
    ap.add_argument("--optimizer", default="adamw", choices=sorted(OPTIMIZERS), help="default: the headline AdamW")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"], help="storage type of parameters, gradients and states (the metric is quoted on bf16)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip timing the reference's CUDA back ends on the 1.1 B list (N=1)")
    ap.add_argument("--reduce-grads", action="store_true", help="N>1 with the push exchange: also average the ranks' gradients inside the step kernel")
    ap.add_argument("--exchange", default="auto", choices=["auto", "push", "nccl"], help="N>1: how updated parameters reach the other ranks")
    args = ap.parse_args()
    if args.workload == "gpt-gradient-release":
        run_gradient_release(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
