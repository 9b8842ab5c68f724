"""Host logic of the ZeRO-1 wrapper on CPU: layouts, and a 2-rank gloo run whose sharded result must
equal the unsharded one bit for bit (with a torch optimizer standing in for the CUDA kernels)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from optimi_b200.zero import ALIGN_ELEMS, FlatLayout, ShardedOptimizer


def test_flat_layout_equal_split_covers_everything_once():
    numels = [1000, 7, 4096, 123457, 1]
    for world in (1, 2, 3, 8):
        lay = FlatLayout(numels, world)
        assert lay.total % (ALIGN_ELEMS * world) == 0
        assert all(o % ALIGN_ELEMS == 0 for o in lay.offsets)
        seen = [0] * len(numels)
        sizes = set()
        for r in range(world):
            lo, hi = lay.rank_range(r)
            sizes.add(hi - lo)
            for i, a, b in lay.pieces(r):
                assert 0 <= a < b <= numels[i]
                assert (lay.offsets[i] + a) % 8 == 0 or a == 0
                seen[i] += b - a
        assert seen == numels and len(sizes) == 1


def test_flat_layout_tensor_split_never_cuts_a_tensor():
    numels = [500_000, 4096, 300_000, 300_000, 4096, 900_000, 16]
    for world in (2, 4):
        lay = FlatLayout(numels, world, split_on_tensors=True)
        owners = {}
        for r in range(world):
            for i, a, b in lay.pieces(r):
                assert (a, b) == (0, numels[i])
                owners[i] = r
        assert sorted(owners) == list(range(len(numels)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, split_on_tensors, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        shapes = [(33, 65), (129,), (1024, 3), (7,), (2000,)]
        params = [torch.nn.Parameter(torch.randn(s, generator=g)) for s in shapes]
        ref = [torch.nn.Parameter(p.detach().clone()) for p in params]
        sharded = ShardedOptimizer(torch.optim.AdamW, params, split_on_tensors=split_on_tensors, lr=1e-2, weight_decay=0.1)
        plain = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1)
        for step in range(4):
            grads = [torch.randn(s, generator=g) for s in shapes]
            for p, r, gr in zip(params, ref, grads):
                p.grad, r.grad = gr.clone(), gr.clone()
            sharded.step()
            plain.step()
            sharded.zero_grad()
        ok = all(torch.equal(p.detach(), r.detach()) for p, r in zip(params, ref))
        n_local = sharded.local_elements()
        gathered = [None] * world
        dist.all_gather_object(gathered, n_local)
        sd = sharded.state_dict()
        assert sd["rank"] == rank and sd["world"] == world
        sharded.load_state_dict(sd)
        if rank == 0:
            out.put((ok, gathered, sum(p.numel() for p in params)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("split_on_tensors", [False, True])
def test_two_ranks_match_unsharded(split_on_tensors):
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, split_on_tensors, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    ok, local_sizes, total = out.get()
    assert ok, "sharded parameters differ from the unsharded run"
    assert sum(local_sizes) == total
    if not split_on_tensors:
        assert abs(local_sizes[0] - local_sizes[1]) <= 2 * ALIGN_ELEMS * 6


def _ckpt_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        shapes = [(33, 65), (129,), (1024, 3), (7,), (2000,)]
        init = [torch.randn(s, generator=g) for s in shapes]
        grads = [[torch.randn(s, generator=g) for s in shapes] for _ in range(6)]
        kw = dict(lr=1e-2, weight_decay=0.1)

        def step(opt, params, gs):
            for p, gr in zip(params, gs):
                p.grad = gr.clone()
            opt.step()

        ref_params = [torch.nn.Parameter(t.clone()) for t in init]
        ref = torch.optim.AdamW(ref_params, **kw)
        params = [torch.nn.Parameter(t.clone()) for t in init]
        sharded = ShardedOptimizer(torch.optim.AdamW, params, **kw)
        for gs in grads[:3]:
            step(ref, ref_params, gs)
            step(sharded, params, gs)
        full = sharded.consolidated_state_dict()
        want = ref.state_dict()
        same_layout = sorted(full["state"]) == sorted(want["state"]) and all(
            sorted(full["state"][i]) == sorted(want["state"][i]) for i in want["state"]
        )
        same_values = all(
            torch.equal(torch.as_tensor(full["state"][i][k]).cpu(), torch.as_tensor(want["state"][i][k]).cpu())
            for i in want["state"] for k in want["state"][i]
        )
        # the consolidated dict loads into a plain optimizer ...
        plain_params = [torch.nn.Parameter(p.detach().clone()) for p in params]
        plain = torch.optim.AdamW(plain_params, **kw)
        plain.load_state_dict(full)
        # ... and into a fresh sharded one; all three continue identically
        params2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
        sharded2 = ShardedOptimizer(torch.optim.AdamW, params2, **kw)
        sharded2.load_consolidated_state_dict(full)
        for gs in grads[3:]:
            step(ref, ref_params, gs)
            step(plain, plain_params, gs)
            step(sharded2, params2, gs)
        cont = all(torch.equal(a.detach(), b.detach()) and torch.equal(a.detach(), c.detach()) for a, b, c in zip(ref_params, plain_params, params2))
        if rank == 0:
            out.put((same_layout, same_values, cont))
    finally:
        dist.destroy_process_group()


def test_consolidated_state_dict_round_trip():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_ckpt_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    same_layout, same_values, cont = out.get()
    assert same_layout, "consolidated state dict has another layout than the unsharded optimizer's"
    assert same_values, "consolidated state differs from the unsharded optimizer's"
    assert cont, "runs continued from the consolidated checkpoint diverge"


def _mismatch_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 1 was handed a model with one layer of another width: a host-made fault
        shapes = [(33, 65), (129,), (1024, 3)] if rank == 0 else [(33, 65), (130,), (1024, 3)]
        params = [torch.nn.Parameter(torch.zeros(s)) for s in shapes]
        before = [p.data_ptr() for p in params]
        try:
            ShardedOptimizer(torch.optim.AdamW, params, lr=1e-2)
            verdict = "no error"
        except RuntimeError as exc:
            verdict = str(exc)
        untouched = before == [p.data_ptr() for p in params]  # nothing was re-pointed into a flat buffer
        out.put((rank, verdict, untouched))
    finally:
        dist.destroy_process_group()


def test_ranks_with_different_parameter_lists_are_refused_before_anything_is_built():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_mismatch_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, verdict, untouched in got:
        assert "different parameter lists" in verdict, f"rank {rank}: {verdict}"
        assert untouched, f"rank {rank}: parameters were moved although the ranks disagree"


def _groups_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        shapes = [(33, 65), (129,), (1024, 3), (7,), (2000,)]
        dtypes = [torch.float32, torch.float32, torch.float64, torch.float32, torch.float64]
        init = [torch.randn(s, generator=g).to(d) for s, d in zip(shapes, dtypes)]

        def groups(ps):  # two groups with their own options, two dtypes running across both
            return [{"params": [ps[1], ps[3]], "weight_decay": 0.0}, {"params": [ps[0], ps[2], ps[4]], "weight_decay": 0.1, "lr": 3e-2}]

        params = [torch.nn.Parameter(t.clone()) for t in init]
        ref = [torch.nn.Parameter(t.clone()) for t in init]
        sharded = ShardedOptimizer(torch.optim.AdamW, groups(params), lr=1e-2)
        plain = torch.optim.AdamW(groups(ref), lr=1e-2)
        assert len(sharded.buckets) == 2 and len(sharded.param_groups) == 2
        assert sharded.param_groups[1]["lr"] == 3e-2 and sharded.param_groups[0]["weight_decay"] == 0.0
        for step in range(4):
            for p, r in zip(params, ref):
                gr = torch.randn(p.shape, generator=g).to(p.dtype)
                p.grad, r.grad = gr.clone(), gr.clone()
            sharded.step()
            plain.step()
        same = all(torch.equal(p.detach(), r.detach()) for p, r in zip(params, ref))
        full, want = sharded.consolidated_state_dict(), plain.state_dict()
        layout = [g_["params"] for g_ in full["param_groups"]] == [g_["params"] for g_ in want["param_groups"]]
        values = all(
            torch.equal(torch.as_tensor(full["state"][i][k]).cpu(), torch.as_tensor(want["state"][i][k]).cpu())
            for i in want["state"] for k in want["state"][i]
        )
        # and back into a fresh sharded optimizer, which then continues like the plain one
        params2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
        sharded2 = ShardedOptimizer(torch.optim.AdamW, groups(params2), lr=1e-2)
        sharded2.load_consolidated_state_dict(full)
        for p, r in zip(params2, ref):
            gr = torch.randn(p.shape, generator=g).to(p.dtype)
            p.grad, r.grad = gr.clone(), gr.clone()
        sharded2.step()
        plain.step()
        cont = all(torch.equal(p.detach(), r.detach()) for p, r in zip(params2, ref))
        identical = sharded2.check_replicas()["ranks_identical"]
        if rank == 0:
            out.put((same, layout, values, cont, identical))
    finally:
        dist.destroy_process_group()


def test_param_groups_and_mixed_dtypes_match_unsharded():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_groups_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        same, layout, values, cont, identical = out.get(timeout=120)
    finally:
        for p in procs:
            p.join(60)
            if p.is_alive():
                p.terminate()
    assert same, "sharded parameters differ from the unsharded run"
    assert layout, "consolidated param_groups number the parameters differently from the unsharded optimizer"
    assert values, "consolidated state differs from the unsharded optimizer's"
    assert cont, "the run continued from the consolidated checkpoint diverges"
    assert identical, "check_replicas() reports differing ranks"


def test_layout_digest_covers_what_decides_the_layout():
    from optimi_b200.zero import _as_groups, layout_digest

    a = [torch.zeros(10), torch.zeros(3, 4), torch.zeros(5, dtype=torch.float64)]
    base = layout_digest(_as_groups(a), 2, "AdamW", False, "push")
    assert base == layout_digest(_as_groups([torch.ones(10), torch.ones(3, 4), torch.ones(5, dtype=torch.float64)]), 2, "AdamW", False, "push")
    different = [
        layout_digest(_as_groups([torch.zeros(11), a[1], a[2]]), 2, "AdamW", False, "push"),  # a size
        layout_digest(_as_groups([a[0], a[1], torch.zeros(5)]), 2, "AdamW", False, "push"),  # a dtype
        layout_digest(_as_groups([{"params": a[:1]}, {"params": a[1:]}]), 2, "AdamW", False, "push"),  # the grouping
        layout_digest(_as_groups(a), 4, "AdamW", False, "push"),  # the world size
        layout_digest(_as_groups(a), 2, "StableAdamW", True, "push"),  # optimizer and split mode
        layout_digest(_as_groups(a), 2, "AdamW", False, "nccl"),  # the exchange
    ]
    assert base not in different and len(set(different)) == len(different)
