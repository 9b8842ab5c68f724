"""ZeRO-1 sharding on real GPUs (needs at least two): whatever way the updated parameters travel,
every rank must end up with exactly the parameters of an unsharded run.

All cases of this file run inside ONE set of worker processes (one per GPU, spawned once per test
session by the `zero_results` fixture): process start-up, NCCL initialisation and the symmetric
memory handshake dominate the cost of a case, and a machine with eight GPUs is not kept waiting
thirteen times.  Each test then only looks up its own case's verdict.

Two ranks by default; ``OPTIMI_TEST_WORLD=4`` (or 8) on a machine with that many GPUs runs the same
cases over more ranks (the gradient-mean kernels are compiled per rank bound 2, 4, 8).  The session takes
about half a minute over two ranks and a minute and a quarter over four (start-up and the symmetric-memory
handshakes grow with the rank count); give eight ranks ten minutes.
"""

import datetime
import io
import os
import queue
import socket
import sys
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPES = [(257, 129), (4096,), (1000, 333), (7,), (65536,), (300, 1024)]


def _host_params(gen, shapes=SHAPES, dtype=torch.bfloat16):
    return [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in shapes]


def _same(params, ref):
    return all(torch.equal(p.detach(), r.detach()) for p, r in zip(params, ref))


# ---------------------------------------------------------------------------------------------
# cases: each returns "" when it passed, a description of what differs otherwise ("SKIP: ..." to skip)
# ---------------------------------------------------------------------------------------------
def case_sharded_equals_unsharded(rank, world, cname, kw, exchange):
    import optimi_b200
    from optimi_b200.zero import ShardedOptimizer

    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    host = _host_params(g)
    params = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
    ref = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
    cls = getattr(optimi_b200, cname)
    sharded = ShardedOptimizer(cls, params, exchange=exchange, **kw)
    if sharded.exchange != exchange:
        return f"asked for exchange={exchange}, got {sharded.exchange}"
    plain = cls(ref, **kw)
    for _ in range(5):
        grads = [(torch.randn(s, generator=g) * 1e-3).to(torch.bfloat16).to(dev) for s in SHAPES]
        for p, r, gr in zip(params, ref, grads):
            p.grad, r.grad = gr.clone(), gr.clone()
        sharded.step()
        plain.step()
        sharded.zero_grad()
    torch.cuda.synchronize()
    if not _same(params, ref):
        return "sharded parameters differ from the unsharded run"
    check = sharded.check_replicas()
    return "" if check["ranks_identical"] else "check_replicas() reports differing ranks after identical steps"


def case_fused_gradient_mean(rank, world, cname, kw):
    """reduce-scatter + step + all-gather in one kernel: equals an unsharded step on the mean gradient."""
    import optimi_b200
    from optimi_b200.zero import ShardedOptimizer

    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    host = _host_params(g)
    params = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
    ref = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
    cls = getattr(optimi_b200, cname)
    sharded = ShardedOptimizer(cls, params, exchange="push", reduce_grads=True, **kw)
    plain = cls(ref, **kw)
    for _ in range(4):
        # every rank draws the gradients of ALL ranks (same generator), keeps its own, and the
        # unsharded run steps with their fp32 mean rounded once
        per_rank = [[(torch.randn(s, generator=g) * 1e-3).to(torch.bfloat16) for s in SHAPES] for _ in range(world)]
        sharded.attach_grads()
        for p, gr in zip(params, per_rank[rank]):
            p.grad.copy_(gr.to(dev))
        for i, r in enumerate(ref):
            acc = per_rank[0][i].float()
            for other in per_rank[1:]:
                acc = acc + other[i].float()
            r.grad = (acc * (1.0 / world)).to(torch.bfloat16).to(dev)
        sharded.step()
        plain.step()
        sharded.zero_grad()
    torch.cuda.synchronize()
    return "" if _same(params, ref) else "fused gradient mean + step differs from the unsharded run on the mean gradient"


def _toy_model(dev):
    """A GPT-shaped toy after optimi's canonical preparation: `to_low_precision` keeps the embedding in
    float32 and `param_groups_weight_decay` splits off biases and norm weights — two groups, two dtypes."""
    import optimi_b200

    torch.manual_seed(0)
    model = torch.nn.Sequential(
        torch.nn.Embedding(500, 96), torch.nn.Linear(96, 384), torch.nn.LayerNorm(384), torch.nn.Linear(384, 96), torch.nn.LayerNorm(96)
    )
    optimi_b200.to_low_precision(model, device=dev)
    return model


def case_param_groups_mixed_dtypes_and_clip(rank, world, exchange, clip):
    """What optimi users actually pass: two param groups x two dtypes, optionally with gradient-norm clipping;
    sharded == unsharded, bit for bit."""
    import optimi_b200
    from optimi_b200.zero import ShardedOptimizer

    dev = torch.device("cuda", rank)
    model, twin = _toy_model(dev), _toy_model(dev)
    kw = dict(lr=1e-3, betas=(0.9, 0.99), eps=1e-6)
    sharded = ShardedOptimizer(optimi_b200.AdamW, optimi_b200.param_groups_weight_decay(model, weight_decay=1e-2), exchange=exchange, **kw)
    plain = optimi_b200.AdamW(optimi_b200.param_groups_weight_decay(twin, weight_decay=1e-2), **kw)
    if sharded.exchange != exchange:
        return f"asked for exchange={exchange}, got {sharded.exchange}"
    if len(sharded.buckets) != 2 or len(sharded.param_groups) != 2:
        return f"expected two dtype buckets and two groups, got {len(sharded.buckets)} and {len(sharded.param_groups)}"
    g = torch.Generator().manual_seed(1)
    norms = []
    for it in range(6):
        for p, q in zip(model.parameters(), twin.parameters()):
            # large gradients on odd steps so that the clip coefficient is below one there
            gr = (torch.randn(p.shape, generator=g) * (1e-3 if it % 2 == 0 else 3.0)).to(p.dtype).to(dev)
            p.grad, q.grad = gr.clone(), gr.clone()
        if clip:
            norms.append((sharded.clip_grad_norm(1.0), plain.clip_grad_norm(1.0)))
        sharded.step()
        plain.step()
        sharded.zero_grad()
    torch.cuda.synchronize()
    for a, b in norms:
        if not torch.equal(a, b):
            return f"total gradient norm differs: sharded {a.item()!r}, unsharded {b.item()!r}"
    for (name, p), q in zip(model.named_parameters(), twin.parameters()):
        if not torch.equal(p.detach(), q.detach()):
            return f"{name} ({p.dtype}) differs from the unsharded run"
    return ""


def case_replica_check_sees_a_flipped_bit(rank, world):
    """Host-made failure: one rank's copy of a parameter is changed by one bit between steps (a plain tensor
    write, no GPU fault); `check_replicas` must report it on every rank."""
    import optimi_b200
    from optimi_b200.zero import ShardedOptimizer

    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    params = [torch.nn.Parameter(h.clone().to(dev)) for h in _host_params(g)]
    sharded = ShardedOptimizer(optimi_b200.AdamW, params, exchange="nccl", lr=1e-3)
    for p in params:
        p.grad = torch.full_like(p, 1e-3)
    sharded.step()
    if not sharded.check_replicas()["ranks_identical"]:
        return "ranks differ right after a step"
    if rank == world - 1:
        bits = params[2].data.view(torch.int16).view(-1)
        bits[12345] ^= 1
    seen = sharded.check_replicas()["ranks_identical"]
    return "a flipped bit on one rank went unnoticed" if seen else ""


def case_step_in_pieces(rank, world, exchange):
    """begin_step / step_groups / end_step over three parameter groups equals one step() of an unsharded optimizer."""
    import optimi_b200
    from optimi_b200.zero import ShardedOptimizer

    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    host = _host_params(g)
    params = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
    ref = [torch.nn.Parameter(h.clone().to(dev)) for h in host]

    def groups(ps):
        return [{"params": ps[0:2]}, {"params": ps[2:3], "weight_decay": 0.0}, {"params": ps[3:]}]

    kw = dict(lr=3e-4, weight_decay=1e-2)
    sharded = ShardedOptimizer(optimi_b200.AdamW, groups(params), exchange=exchange, **kw)
    plain = optimi_b200.AdamW(groups(ref), **kw)
    for _ in range(4):
        grads = [(torch.randn(s, generator=g) * 1e-3).to(torch.bfloat16).to(dev) for s in SHAPES]
        for p, r, gr in zip(params, ref, grads):
            p.grad, r.grad = gr.clone(), gr.clone()
        sharded.begin_step()
        for gi in (2, 0, 1):  # any order, each group once
            sharded.step_groups([gi])
        sharded.end_step()
        plain.step()
        sharded.zero_grad()
    torch.cuda.synchronize()
    return "" if _same(params, ref) else "a step in pieces differs from the unsharded step"


def _reference_package():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        return None
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import optimi  # the unmodified reference

    return optimi


def case_checkpoint_round_trip_with_reference(rank, world, cname, kw, exact):
    """The reference's own checkpoint test (tests/runner.py:244-251: save, torch.load(weights_only=True), fresh
    optimizer, load, continue) across the two implementations: a sharded optimi_b200 run's consolidated
    checkpoint continues in the reference's optimizer, and a reference checkpoint continues in a sharded
    optimi_b200 run; both must land where an uninterrupted unsharded optimi_b200 run lands."""
    import optimi_b200
    from optimi_b200.zero import ShardedOptimizer

    optimi = _reference_package()
    if optimi is None:
        return "SKIP: reference package not present beside the repository"
    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    host = _host_params(g)
    grads = [[(torch.randn(s, generator=g) * 1e-3).to(torch.bfloat16).to(dev) for s in SHAPES] for _ in range(8)]
    cls, ref_cls = getattr(optimi_b200, cname), getattr(optimi, cname)

    def fresh():
        return [torch.nn.Parameter(h.clone().to(dev)) for h in host]

    def run(opt, params, gs):
        for step_grads in gs:
            for p, gr in zip(params, step_grads):
                p.grad = gr.clone()  # the reference's foreach path uses its gradients as scratch
            opt.step()

    def through_a_file(sd):
        buf = io.BytesIO()
        torch.save(sd, buf)
        buf.seek(0)
        return torch.load(buf, weights_only=True)

    def close(a, b):
        if exact:
            return torch.equal(a, b)
        scale = torch.maximum(a.float().abs(), b.float().abs()).clamp_min(1e-3)
        return not bool(((a.float() - b.float()).abs() > scale * 2.0**-7).any())  # 1 bf16 ulp

    straight = fresh()
    run(cls(straight, **kw), straight, grads)

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        # sharded optimi_b200 -> reference
        params = fresh()
        sharded = ShardedOptimizer(cls, params, exchange="push", **kw)
        run(sharded, params, grads[:3])
        ckpt = through_a_file(sharded.consolidated_state_dict())
        theirs = [torch.nn.Parameter(p.detach().clone()) for p in params]
        ref_opt = ref_cls(theirs, foreach=True, triton=False, **kw)
        ref_opt.load_state_dict(ckpt)
        run(ref_opt, theirs, grads[3:])
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(zip(theirs, straight)):
            if not close(a.detach(), b.detach()):
                return f"tensor {i}: the reference continued from the sharded checkpoint differs from the uninterrupted run"

        # reference -> sharded optimi_b200
        theirs = fresh()
        ref_opt = ref_cls(theirs, foreach=True, triton=False, **kw)
        run(ref_opt, theirs, grads[:3])
        ckpt = through_a_file(ref_opt.state_dict())
        params = [torch.nn.Parameter(p.detach().clone()) for p in theirs]
        sharded = ShardedOptimizer(cls, params, exchange="nccl", **kw)
        sharded.load_consolidated_state_dict(ckpt)
        run(sharded, params, grads[3:])
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(zip(params, straight)):
            if not close(a.detach(), b.detach()):
                return f"tensor {i}: the sharded run continued from the reference's checkpoint differs from the uninterrupted run"
    return ""


ADAMW = dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True)
CASES = {
    "AdamW-nccl": (case_sharded_equals_unsharded, ("AdamW", ADAMW, "nccl")),
    "AdamW-push": (case_sharded_equals_unsharded, ("AdamW", ADAMW, "push")),
    "Adam-plain-push": (case_sharded_equals_unsharded, ("Adam", dict(lr=3e-4, weight_decay=1e-2, kahan_sum=False), "push")),
    "StableAdamW-nccl": (case_sharded_equals_unsharded, ("StableAdamW", dict(lr=3e-4), "nccl")),
    "StableAdamW-push": (case_sharded_equals_unsharded, ("StableAdamW", dict(lr=3e-4), "push")),
    "Adan-nccl": (case_sharded_equals_unsharded, ("Adan", dict(lr=3e-4, kahan_sum=True), "nccl")),
    "Adan-push": (case_sharded_equals_unsharded, ("Adan", dict(lr=3e-4, kahan_sum=True), "push")),
    "Lion-push": (case_sharded_equals_unsharded, ("Lion", dict(lr=1e-4, weight_decay=0.1), "push")),
    "SGD-push": (case_sharded_equals_unsharded, ("SGD", dict(lr=1e-2, momentum=0.9), "push")),
    "Ranger-push": (case_sharded_equals_unsharded, ("Ranger", dict(lr=3e-4, k=2), "push")),
    "fused-AdamW": (case_fused_gradient_mean, ("AdamW", ADAMW)),
    "fused-Lion": (case_fused_gradient_mean, ("Lion", dict(lr=1e-4))),
    "fused-Adan": (case_fused_gradient_mean, ("Adan", dict(lr=3e-4, kahan_sum=True))),
    "fused-SGD-torch-init": (case_fused_gradient_mean, ("SGD", dict(lr=1e-2, momentum=0.9, dampening=True, torch_init=True))),
    "groups-dtypes-nccl": (case_param_groups_mixed_dtypes_and_clip, ("nccl", False)),
    "groups-dtypes-push": (case_param_groups_mixed_dtypes_and_clip, ("push", False)),
    "groups-dtypes-clip-nccl": (case_param_groups_mixed_dtypes_and_clip, ("nccl", True)),
    "groups-dtypes-clip-push": (case_param_groups_mixed_dtypes_and_clip, ("push", True)),
    "replica-check": (case_replica_check_sees_a_flipped_bit, ()),
    "step-in-pieces-nccl": (case_step_in_pieces, ("nccl",)),
    "step-in-pieces-push": (case_step_in_pieces, ("push",)),
    "checkpoint-reference-Adan": (case_checkpoint_round_trip_with_reference, ("Adan", dict(lr=3e-4, kahan_sum=True), True)),
    "checkpoint-reference-StableAdamW": (case_checkpoint_round_trip_with_reference, ("StableAdamW", dict(lr=3e-4), False)),
}


# ---------------------------------------------------------------------------------------------
# one set of ranks runs every case
# ---------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case_ids, out):
    # plain peer loads/stores and NCCL without NVLS: a rank that dies must not leave multicast bindings behind
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=240))  # fmt: skip
    results = {}
    try:
        for cid in case_ids:
            fn, args = CASES[cid]
            try:
                msg = fn(rank, world, *args)
            except Exception as exc:  # reported as this case's failure; the ranks meet again right below
                msg = f"rank {rank}: {type(exc).__name__}: {exc}"
            msgs = [None] * world
            dist.all_gather_object(msgs, msg)
            results[cid] = sorted({m for m in msgs if m})
            torch.cuda.synchronize()
        if rank == 0:
            out.put(results)
    finally:
        dist.destroy_process_group()


@pytest.fixture(scope="module")
def zero_results():
    world = int(os.environ.get("OPTIMI_TEST_WORLD", "2"))
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, list(CASES), out)) for r in range(world)]
    for p in procs:
        p.start()
    results = None
    try:
        results = out.get(timeout=900)
    except queue.Empty:
        pass
    finally:
        # never leave a straggler blocked in a collective on a shared GPU
        for p in procs:
            p.join(30 if results is not None else 1)
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
            if p.is_alive():
                p.kill()
                p.join(5)
    if results is None:
        pytest.fail(f"the {world} worker ranks did not report (exit codes {[p.exitcode for p in procs]})")
    return results


@pytest.mark.parametrize("case_id", list(CASES))
def test_zero(zero_results, case_id):
    problems = zero_results.get(case_id)
    assert problems is not None, "the workers never reached this case"
    if problems and all(m.startswith("SKIP:") for m in problems):
        pytest.skip(problems[0][5:].strip())
    assert not problems, "; ".join(problems)
