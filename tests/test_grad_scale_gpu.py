"""Gradient scaling fused into the step: `set_grad_factor` must equal multiplying the gradients first
(`torch._foreach_mul_` arithmetic: fp32 product, one rounding to the storage type) and stepping plainly;
`clip_grad_norm` must produce torch.nn.utils.clip_grad_norm_'s norm and coefficient."""

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(257, 129), (4096,), (1000, 333), (7,), (65536,), (300, 1024)]

CASES = [
    ("AdamW", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True)),
    ("Adam", dict(lr=3e-4, weight_decay=1e-2, kahan_sum=False)),
    ("StableAdamW", dict(lr=3e-4, weight_decay=1e-2)),
    ("Ranger", dict(lr=3e-4, k=2)),
    ("RAdam", dict(lr=3e-4)),
    ("Lion", dict(lr=1e-4, weight_decay=0.1)),
    ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2)),
    ("Adan", dict(lr=3e-4, kahan_sum=True)),
]


def _params(dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter((torch.randn(s, generator=g) * 0.02).to(dtype).cuda()) for s in SHAPES]


def _state_tensors(opt, params):
    return [(k, v) for p in params for k, v in sorted(opt.state[p].items()) if torch.is_tensor(v) and v.is_cuda]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
@pytest.mark.parametrize("cname,kw", CASES, ids=[c[0] for c in CASES])
def test_scaled_step_equals_scaling_then_stepping(cname, kw, dtype):
    import optimi_b200

    cls = getattr(optimi_b200, cname)
    pa, pb = _params(dtype), _params(dtype)
    plain, fused = cls(pa, **kw), cls(pb, **kw)
    factor = torch.zeros(1, dtype=torch.float32, device="cuda")
    fused.set_grad_factor(factor)
    gen = torch.Generator().manual_seed(1)
    for it, f in enumerate([0.37, 1.0, 1.0 / 65536.0, 0.9990234375]):
        factor.fill_(f)
        grads = [(torch.randn(s, generator=gen) * (1e-3 if it != 2 else 60.0)).to(dtype).cuda() for s in SHAPES]
        for p, q, g in zip(pa, pb, grads):
            p.grad = (g.float() * factor).to(dtype)  # fp32 product, one rounding
            q.grad = g.clone()
        plain.step()
        fused.step()
        for q, g in zip(pb, grads):
            assert torch.equal(q.grad, g), "the fused path must leave the gradients alone"
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        assert torch.equal(p.detach(), q.detach())
    for (k, a), (_, b) in zip(_state_tensors(plain, pa), _state_tensors(fused, pb)):
        assert torch.equal(a, b), k
    # switching it off again
    fused.set_grad_factor(None)
    for p, q in zip(pa, pb):
        p.grad = torch.ones_like(p) * 1e-3
        q.grad = torch.ones_like(q) * 1e-3
    plain.step()
    fused.step()
    for p, q in zip(pa, pb):
        assert torch.equal(p.detach(), q.detach())


def _ulp(x: torch.Tensor, dtype) -> float:
    bits = {torch.bfloat16: 8, torch.float16: 11, torch.float32: 24}[dtype]
    return float(2.0 ** (torch.floor(torch.log2(x.abs().float().clamp_min(1e-30))) - (bits - 1)))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16], ids=["bf16", "f32", "f16"])
@pytest.mark.parametrize("max_norm", [0.05, 1.0, 1e4])
def test_clip_factor_matches_torch(dtype, max_norm):
    import optimi_b200

    params = _params(dtype)
    gen = torch.Generator().manual_seed(3)
    shadow = []
    for p in params:
        p.grad = (torch.randn(p.shape, generator=gen) * 1e-2).to(dtype).cuda()
        s = torch.nn.Parameter(p.detach().clone())
        s.grad = p.grad.clone()
        shadow.append(s)
    opt = optimi_b200.AdamW(params, lr=1e-3)
    total = opt.clip_grad_norm(max_norm)
    factor = opt._grad_factor.clone()
    ref_total = torch.nn.utils.clip_grad_norm_(shadow, max_norm, foreach=True)
    ref_factor = torch.clamp(max_norm / (ref_total + 1e-6), max=1.0)
    assert ref_total.dtype == dtype
    # sums are taken in another order (and in double), so allow one unit of the storage type
    assert abs(float(total) - float(ref_total)) <= _ulp(ref_total, dtype)
    assert abs(float(factor) - float(ref_factor)) <= _ulp(ref_factor, dtype)
    if max_norm == 1e4:
        assert float(factor) == 1.0
    else:
        assert float(factor) < 1.0
    # the gradients are untouched by the fused clip, scaled in place by torch's
    for p, s in zip(params, shadow):
        if float(factor) == float(ref_factor):
            assert torch.equal((p.grad.float() * factor).to(dtype), s.grad)


def test_clip_then_step_equals_scaling_with_the_same_factor_then_stepping():
    import optimi_b200

    pa, pb = _params(torch.bfloat16), _params(torch.bfloat16)
    plain = optimi_b200.AdamW(pa, lr=3e-4, weight_decay=1e-2)
    fused = optimi_b200.AdamW(pb, lr=3e-4, weight_decay=1e-2)
    gen = torch.Generator().manual_seed(5)
    for it in range(4):
        grads = [(torch.randn(s, generator=gen) * 1e-2).to(torch.bfloat16).cuda() for s in SHAPES]
        for q, g in zip(pb, grads):
            q.grad = g.clone()
        norm = fused.clip_grad_norm(0.5)
        factor = fused._grad_factor.clone()
        assert 0.0 < float(factor) < 1.0 and float(norm) > 0.5
        for p, g in zip(pa, grads):
            p.grad = (g.float() * factor).to(torch.bfloat16)
        plain.step()
        fused.step()
        assert fused._grad_factor is None  # the coefficient belonged to that step only
    for p, q in zip(pa, pb):
        assert torch.equal(p.detach(), q.detach())


def test_factor_inside_a_cuda_graph():
    import optimi_b200

    pa, pb = _params(torch.bfloat16), _params(torch.bfloat16)
    eager = optimi_b200.AdamW(pa, lr=3e-4)
    captured = optimi_b200.AdamW(pb, lr=3e-4)
    gen = torch.Generator().manual_seed(7)

    def draw():
        return [(torch.randn(s, generator=gen) * 1e-2).to(torch.bfloat16).cuda() for s in SHAPES]

    first = draw()
    for p, q, g in zip(pa, pb, first):
        p.grad, q.grad = g.clone(), g.clone()
    eager.step()
    captured.step()
    graph = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.graph(graph):
        captured.clip_grad_norm(0.5)  # the norm kernels are captured too; their coefficient feeds the captured step
        captured.step()
    graph.instantiate()
    for it in range(4):
        grads = draw()
        for p, q, g in zip(pa, pb, grads):
            p.grad = g.clone()
            q.grad.copy_(g)
        eager.clip_grad_norm(0.5)
        eager.step()
        captured.update_graph(graph)
        graph.replay()
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        assert torch.equal(p.detach(), q.detach())


def test_gradient_release_applies_the_factor():
    """Hooks that step during backward unscale a loss scale on the fly, accumulation micro-steps included."""
    import optimi_b200
    from optimi_b200 import prepare_for_gradient_release, remove_gradient_release

    torch.manual_seed(0)
    model_a = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).cuda().bfloat16()
    model_b = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).cuda().bfloat16()
    model_b.load_state_dict(model_a.state_dict())
    manual = optimi_b200.AdamW(model_a.parameters(), lr=1e-3, gradient_release=True)  # stepped by hand, no hooks
    hooked = optimi_b200.AdamW(model_b.parameters(), lr=1e-3, gradient_release=True)
    prepare_for_gradient_release(model_b, hooked)
    factor = torch.full((1,), 1.0 / 128.0, dtype=torch.float32, device="cuda")
    hooked.set_grad_factor(factor)
    x = torch.randn(16, 64, device="cuda", dtype=torch.bfloat16)
    for it in range(4):
        manual.optimizer_accumulation = hooked.optimizer_accumulation = it % 2 == 0
        (model_a(x).float().square().mean() * 128.0).backward()  # a "loss scale" of 128
        for p in model_a.parameters():
            p.grad = (p.grad.float() * factor).to(torch.bfloat16)
            manual.step(param=p)
            manual.zero_grad(param=p)
        (model_b(x).float().square().mean() * 128.0).backward()  # stepped by the hooks, unscaled as the kernels load
    torch.cuda.synchronize()
    remove_gradient_release(model_b)
    for p, q in zip(model_a.parameters(), model_b.parameters()):
        assert torch.equal(p.detach(), q.detach())
    for p, q in zip(model_a.parameters(), model_b.parameters()):
        for k in ("exp_avg", "exp_avg_sq", "kahan_comp"):
            assert torch.equal(manual.state[p][k], hooked.state[q][k]), k
    with pytest.raises(RuntimeError, match="gradient_release"):
        hooked.clip_grad_norm(1.0)


@pytest.mark.parametrize("max_norm", [0.05, 1e4])
def test_clip_factor_over_mixed_dtypes_matches_torch(max_norm):
    """float32 embeddings beside a bfloat16 body (what `to_low_precision` leaves): per-tensor norms in each tensor's
    dtype, the total norm and the coefficient in float32, as torch.nn.utils.clip_grad_norm_ promotes them; then a step
    with the coefficient equals scaling the gradients (each in its own dtype) and stepping plainly."""
    import optimi_b200

    gen = torch.Generator().manual_seed(9)
    dtypes = [torch.float32, torch.bfloat16, torch.bfloat16, torch.float32, torch.bfloat16]
    shapes = [(300, 64), (257, 129), (4096,), (7,), (1000, 33)]
    host = [(torch.randn(s, generator=gen) * 0.02).to(d) for s, d in zip(shapes, dtypes)]
    fused = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    plain = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    shadow = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    for p, q, s in zip(fused, plain, shadow):
        g = (torch.randn(p.shape, generator=gen) * 1e-2).to(p.dtype).cuda()
        p.grad, s.grad = g.clone(), g.clone()
    opt = optimi_b200.AdamW(fused, lr=1e-3)
    total = opt.clip_grad_norm(max_norm)
    factor = opt._grad_factor.clone()
    ref_total = torch.nn.utils.clip_grad_norm_(shadow, max_norm, foreach=True)
    ref_factor = torch.clamp(max_norm / (ref_total + 1e-6), max=1.0)
    assert ref_total.dtype == torch.float32
    assert abs(float(total) - float(ref_total)) <= 2 * _ulp(ref_total, torch.float32) + 1e-6 * float(ref_total)
    assert abs(float(factor) - float(ref_factor)) <= 1e-6 * float(ref_factor) + 1e-12
    assert (float(factor) == 1.0) == (max_norm == 1e4)
    # stepping with the coefficient == scaling each gradient in its own dtype, then stepping
    ref_opt = optimi_b200.AdamW(plain, lr=1e-3)
    for p, q in zip(fused, plain):
        q.grad = (p.grad.float() * factor).to(p.dtype)
    opt.step()
    ref_opt.step()
    torch.cuda.synchronize()
    for p, q in zip(fused, plain):
        assert torch.equal(p.detach(), q.detach()), f"{p.dtype} tensor {tuple(p.shape)} differs"
