"""Gradient release and optimizer accumulation on a real backward pass.

A small MLP is trained with `prepare_for_gradient_release` hooks; every gradient the hooks consume is
recorded and replayed through the CPU oracle's per-parameter step (the reference's `_single_param_*`
semantics: per-parameter step counters that also advance on accumulation micro-steps,
optimi/adam.py:183-208, 261).  Parameters must match bit for bit, with the steps on the backward
stream or on a side stream.
"""

import warnings

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


def make_model(dtype):
    torch.manual_seed(0)
    model = nn.Sequential(nn.LayerNorm(64), nn.Linear(64, 256), nn.Mish(), nn.Linear(256, 128), nn.GELU(), nn.Linear(128, 1))
    return model.to(device="cuda", dtype=dtype)


CASES = [
    ("adamw", "AdamW", dict(lr=1e-3, weight_decay=1e-2), torch.bfloat16),
    ("adamw", "AdamW", dict(lr=1e-3, weight_decay=1e-2), torch.float32),
    ("lion", "Lion", dict(lr=1e-4, weight_decay=0.1), torch.bfloat16),
    ("sgd", "SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2), torch.bfloat16),
    ("adan", "Adan", dict(lr=1e-3, kahan_sum=True), torch.bfloat16),
    ("radam", "RAdam", dict(lr=1e-3), torch.float32),
    ("ranger", "Ranger", dict(lr=1e-3, k=3), torch.float32),
]


@pytest.mark.parametrize("oname,cname,kw,dtype", CASES, ids=[f"{c[0]}-{str(c[3]).split('.')[-1]}" for c in CASES])
@pytest.mark.parametrize("side_stream", [False, True], ids=["backward-stream", "side-stream"])
@pytest.mark.parametrize("accumulate", [False, True], ids=["every-step", "accumulate-4"])
def test_hooks_match_oracle(oname, cname, kw, dtype, side_stream, accumulate):
    import optimi_b200
    from oracle.port import OracleOptimizer

    model = make_model(dtype)
    params = [p for p in model.parameters()]
    host0 = [p.detach().cpu().clone() for p in params]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = getattr(optimi_b200, cname)(params, gradient_release=True, **kw)
    opt.use_release_stream(bool(side_stream))  # explicit either way: prepare_for_gradient_release would default to a side stream

    recorded = []  # (iteration, param index, grad)
    index = {id(p): i for i, p in enumerate(params)}
    it_box = [0]
    for p in params:  # record before the release hook consumes the gradient
        p.register_post_accumulate_grad_hook(lambda q: recorded.append((it_box[0], index[id(q)], q.grad.detach().cpu().clone())))
    optimi_b200.prepare_for_gradient_release(model, opt, ignore_existing_hooks=True)

    g = torch.Generator(device="cuda").manual_seed(1)
    iters = 12
    for it in range(iters):
        it_box[0] = it
        opt.optimizer_accumulation = accumulate and (it % 4 != 3)
        x = torch.randn(32, 64, device="cuda", dtype=dtype, generator=g)
        loss = model(x).float().pow(2).mean()
        loss.backward()
        # a plain step / zero_grad after a released backward is a harmless no-op
        assert all(p.grad is None for p in params)
        if it % 5 == 0:
            opt.step()
            opt.zero_grad()
    torch.cuda.synchronize()
    optimi_b200.remove_gradient_release(model)

    oracle = OracleOptimizer(oname, [h.clone() for h in host0], **kw)
    for it, i, grad in recorded:
        oracle.step_param(i, grad.clone(), accumulate=accumulate and (it % 4 != 3))
    for i, p in enumerate(params):
        got, want = p.detach().cpu(), oracle.params[i]
        assert torch.equal(got, want), f"param {i}: max diff {(got.float() - want.float()).abs().max().item()}"


def test_hooks_equal_whole_model_step_when_not_accumulating():
    """Without accumulation every parameter's counter equals the group counter, so released steps and
    one whole-list step per iteration give identical parameters."""
    import optimi_b200

    results = []
    for release in (False, True):
        model = make_model(torch.bfloat16)
        opt = optimi_b200.AdamW(model.parameters(), lr=1e-3, gradient_release=release)
        if release:
            optimi_b200.prepare_for_gradient_release(model, opt)
        g = torch.Generator(device="cuda").manual_seed(1)
        for _ in range(8):
            x = torch.randn(32, 64, device="cuda", dtype=torch.bfloat16, generator=g)
            model(x).float().pow(2).mean().backward()
            if not release:
                opt.step()
                opt.zero_grad()
        torch.cuda.synchronize()
        results.append([p.detach().clone() for p in model.parameters()])
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_state_dict_round_trip_continues_identically():
    """save -> load into a fresh optimizer -> continue: same parameters as an uninterrupted run
    (the reference's checkpoint test, tests/runner.py:244-251)."""
    import io

    import optimi_b200

    def run(interrupt):
        model = make_model(torch.bfloat16)
        opt = optimi_b200.StableAdamW(model.parameters(), lr=1e-3)
        g = torch.Generator(device="cuda").manual_seed(3)
        for it in range(10):
            if interrupt and it == 5:
                buf = io.BytesIO()
                torch.save(opt.state_dict(), buf)
                buf.seek(0)
                opt = optimi_b200.StableAdamW(model.parameters(), lr=1e-3)
                opt.load_state_dict(torch.load(buf, weights_only=True))
            x = torch.randn(32, 64, device="cuda", dtype=torch.bfloat16, generator=g)
            model(x).float().pow(2).mean().backward()
            opt.step()
            opt.zero_grad()
        torch.cuda.synchronize()
        return [p.detach().clone() for p in model.parameters()]

    for a, b in zip(run(False), run(True)):
        assert torch.equal(a, b)
