"""ZeRO-1 sharding on real GPUs (needs at least two): the sharded step + NCCL all-gather must leave
every rank with exactly the parameters of an unsharded run.

The tests run two ranks by default; ``OPTIMI_TEST_WORLD=4`` (or 8) on a machine with that many GPUs
runs the same cases over more ranks (the gradient-mean kernels are compiled per rank bound 2, 4, 8)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _world():
    world = int(os.environ.get("OPTIMI_TEST_WORLD", "2"))
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    return world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, cname, kw, exchange, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import optimi_b200
        from optimi_b200.zero import ShardedOptimizer

        dev = torch.device("cuda", rank)
        g = torch.Generator().manual_seed(0)
        shapes = [(257, 129), (4096,), (1000, 333), (7,), (65536,), (300, 1024)]
        host = [(torch.randn(s, generator=g) * 0.02).to(torch.bfloat16) for s in shapes]
        params = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
        ref = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
        cls = getattr(optimi_b200, cname)
        sharded = ShardedOptimizer(cls, params, exchange=exchange, **kw)
        assert sharded.exchange == exchange
        plain = cls(ref, **kw)
        for _ in range(5):
            grads = [(torch.randn(s, generator=g) * 1e-3).to(torch.bfloat16).to(dev) for s in shapes]
            for p, r, gr in zip(params, ref, grads):
                p.grad, r.grad = gr.clone(), gr.clone()
            sharded.step()
            plain.step()
            sharded.zero_grad()
        torch.cuda.synchronize()
        ok = all(torch.equal(p.detach(), r.detach()) for p, r in zip(params, ref))
        oks = [None] * world
        dist.all_gather_object(oks, ok)
        if rank == 0:
            out.put(all(oks))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cname,kw,exchange", [
    ("AdamW", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True), "nccl"),
    ("AdamW", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True), "push"),
    ("Adam", dict(lr=3e-4, weight_decay=1e-2, kahan_sum=False), "push"),
    ("StableAdamW", dict(lr=3e-4), "nccl"),
    ("StableAdamW", dict(lr=3e-4), "push"),
    ("Adan", dict(lr=3e-4, kahan_sum=True), "nccl"),
    ("Adan", dict(lr=3e-4, kahan_sum=True), "push"),
    ("Lion", dict(lr=1e-4, weight_decay=0.1), "push"),
    ("SGD", dict(lr=1e-2, momentum=0.9), "push"),
    ("Ranger", dict(lr=3e-4, k=2), "push"),
])  # fmt: skip
def test_sharded_step_equals_unsharded(cname, kw, exchange):
    world = _world()
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, cname, kw, exchange, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert out.get(), "sharded parameters differ from the unsharded run"


def _reduce_worker(rank, world, port, cname, kw, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import optimi_b200
        from optimi_b200.zero import ShardedOptimizer

        dev = torch.device("cuda", rank)
        g = torch.Generator().manual_seed(0)
        shapes = [(257, 129), (4096,), (1000, 333), (7,), (65536,), (300, 1024)]
        host = [(torch.randn(s, generator=g) * 0.02).to(torch.bfloat16) for s in shapes]
        params = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
        ref = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
        cls = getattr(optimi_b200, cname)
        sharded = ShardedOptimizer(cls, params, exchange="push", reduce_grads=True, **kw)
        plain = cls(ref, **kw)
        for _ in range(4):
            # every rank draws the gradients of ALL ranks (same generator), keeps its own, and the
            # unsharded run steps with their fp32 mean rounded once
            per_rank = [[(torch.randn(s, generator=g) * 1e-3).to(torch.bfloat16) for s in shapes] for _ in range(world)]
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
        ok = all(torch.equal(p.detach(), r.detach()) for p, r in zip(params, ref))
        oks = [None] * world
        dist.all_gather_object(oks, ok)
        if rank == 0:
            out.put(all(oks))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cname,kw", [("AdamW", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True)), ("Lion", dict(lr=1e-4)),
                                      ("Adan", dict(lr=3e-4, kahan_sum=True))])  # fmt: skip
def test_fused_gradient_mean_step_and_exchange(cname, kw):
    """reduce-scatter + step + all-gather in one kernel: equals an unsharded step on the mean gradient."""
    world = _world()
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_reduce_worker, args=(r, world, port, cname, kw, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert out.get(), "fused gradient mean + step differs from the unsharded run on the mean gradient"
