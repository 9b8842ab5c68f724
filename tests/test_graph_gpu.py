"""A `step()` captured into a CUDA graph and refreshed with `update_graph` before every replay must
leave exactly the parameters and states of the same steps made eagerly, with a learning rate that
changes from step to step."""

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(257, 129), (4096,), (1000, 333), (7,), (65536,), (300, 1024)]

CASES = [
    ("AdamW", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True)),
    ("Adam", dict(lr=3e-4, weight_decay=1e-2, kahan_sum=False)),
    ("StableAdamW", dict(lr=3e-4, weight_decay=1e-2)),
    ("Ranger", dict(lr=3e-4, k=2)),  # every other step launches the lookahead kernel instead: the node's function changes
    ("RAdam", dict(lr=3e-4)),  # the rectified update switches on at step 6
    ("Lion", dict(lr=1e-4, weight_decay=0.1)),
    ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2)),
    ("Adan", dict(lr=3e-4, kahan_sum=True)),
]


def _state_tensors(opt, params):
    out = []
    for p in params:
        for k, v in sorted(opt.state[p].items()):
            if torch.is_tensor(v) and v.is_cuda:
                out.append((k, v))
    return out


def _make(cname, kw, dtype=torch.bfloat16, groups=1):
    import optimi_b200

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(0)
    host = [(torch.randn(s, generator=g) * 0.02).to(dtype) for s in SHAPES]
    params = [torch.nn.Parameter(h.clone().to(dev)) for h in host]
    cls = getattr(optimi_b200, cname)
    if groups == 1:
        return params, cls(params, **kw), g
    half = len(params) // 2
    return params, cls([dict(params=params[:half]), dict(params=params[half:], lr=kw["lr"] * 0.5)], **kw), g


@pytest.mark.parametrize("cname,kw", CASES, ids=[c[0] for c in CASES])
def test_captured_step_equals_eager(cname, kw):
    dev = torch.device("cuda")
    eager_params, eager, gen = _make(cname, kw)
    graph_params, captured, _ = _make(cname, kw)

    def draw():
        return [(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16).to(dev) for s in SHAPES]

    # one eager step on both: the states have to exist before the capture
    first = draw()
    for p, q, gr in zip(eager_params, graph_params, first):
        p.grad, q.grad = gr.clone(), gr.clone()  # q.grad stays where it is from now on (static gradient buffers)
    eager.step()
    captured.step()

    graph = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.graph(graph):
        captured.step()
    graph.instantiate()
    assert len(captured._graph_nodes) >= 1
    steps_before = [int(g["step"]) for g in captured.param_groups if "step" in g]

    for it in range(7):
        lr = kw["lr"] * (1.0 - 0.1 * it)
        for opt in (eager, captured):
            for group in opt.param_groups:
                group["lr"] = lr
        grads = draw()
        for p, q, gr in zip(eager_params, graph_params, grads):
            p.grad = gr.clone()
            q.grad.copy_(gr)
        eager.step()
        captured.update_graph(graph)
        graph.replay()
    torch.cuda.synchronize()

    if steps_before:
        assert [int(g["step"]) for g in captured.param_groups] == [s + 7 for s in steps_before]
        assert [int(g["step"]) for g in captured.param_groups] == [int(g["step"]) for g in eager.param_groups]
    for p, q in zip(eager_params, graph_params):
        assert torch.equal(p.detach(), q.detach())
    for (k, a), (_, b) in zip(_state_tensors(eager, eager_params), _state_tensors(captured, graph_params)):
        assert torch.equal(a, b), k


def test_two_groups_and_two_dtypes_in_one_graph():
    import optimi_b200

    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(1)
    dtypes = [torch.float32, torch.bfloat16, torch.bfloat16, torch.float32, torch.bfloat16, torch.bfloat16]

    def build():
        g = torch.Generator().manual_seed(0)
        ps = [torch.nn.Parameter((torch.randn(s, generator=g) * 0.02).to(dt).to(dev)) for s, dt in zip(SHAPES, dtypes)]
        opt = optimi_b200.AdamW([dict(params=ps[:3]), dict(params=ps[3:], weight_decay=0.0)], lr=1e-3)
        return ps, opt

    def draw():
        return [(torch.randn(s, generator=gen) * 1e-3).to(dt).to(dev) for s, dt in zip(SHAPES, dtypes)]

    pa, eager = build()
    pb, captured = build()
    first = draw()
    for p, q, gr in zip(pa, pb, first):
        p.grad, q.grad = gr.clone(), gr.clone()
    eager.step()
    captured.step()
    graph = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.graph(graph):
        captured.step()
    graph.instantiate()
    assert len(captured._graph_nodes) == 4  # two groups x two storage types
    for it in range(4):
        grads = draw()
        for p, q, gr in zip(pa, pb, grads):
            p.grad = gr.clone()
            q.grad.copy_(gr)
        eager.step()
        captured.update_graph(graph)
        graph.replay()
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        assert torch.equal(p.detach(), q.detach())


def test_plain_launch_into_a_capturing_stream_is_refused():
    """Outside a record bracket the C entry points refuse a capturing stream instead of freezing the
    step's scalars into the graph; the capture itself stays usable."""
    import optimi_b200
    from optimi_b200 import functional as F

    dev = torch.device("cuda")
    p = torch.zeros(1000, device=dev, dtype=torch.bfloat16)
    g = torch.ones_like(p)
    m, v, k = torch.zeros_like(p), torch.zeros_like(p), torch.zeros_like(p)
    step = torch.tensor(0, dtype=torch.int32)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        with pytest.raises(RuntimeError, match="capturing a CUDA graph"):
            F.adam([p], [g], [m], [v], [k], lr=1e-3, beta1=0.9, beta2=0.99, weight_decay=0.0, eps=1e-6, step=step,
                   decouple_wd=True, kahan_sum=True)  # fmt: skip
        p.add_(1.0)  # something for the graph to hold
    graph.replay()
    torch.cuda.synchronize()
    assert float(p[0]) == 1.0 and float(m.abs().max()) == 0.0
    del optimi_b200


def test_capture_needs_existing_states():
    import optimi_b200

    dev = torch.device("cuda")
    p = torch.nn.Parameter(torch.zeros(1000, device=dev, dtype=torch.bfloat16))
    p.grad = torch.ones_like(p)
    opt = optimi_b200.AdamW([p], lr=1e-3)
    graph = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.graph(graph):
        with pytest.raises(RuntimeError, match="one eager step"):
            opt.step()
    with pytest.raises(RuntimeError, match="no captured step"):
        opt.update_graph(graph)
