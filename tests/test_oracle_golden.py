"""Pins the CPU oracle against the golden vectors the unmodified reference produced.

cuda.npz   reference foreach / per-parameter paths run on a B200 (torch 2.11.0+cu128): bit-exact,
           except StableAdamW in float32 where the reference's own reduction order shows up in the
           last bits (1e-6 relative is the stated float32 bar).
cpu_f32    reference foreach path on CPU, float32: 1e-6 relative (CPU ATen fuses and divides
           differently from CUDA ATen; Adan's division by the decay factor reaches 2e-6).
"""

import pytest
import torch

from cases import CASES
from helpers import compare_exact, golden_tensor, load_golden, run_oracle_case

CUDA = load_golden("cuda")
CPU = load_golden("cpu_f32")


def _rel_close(t, w, rtol, atol):
    t, w = t.double().reshape(-1), w.double().reshape(-1)
    return bool(((t - w).abs() <= atol + rtol * w.abs()).all())


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_oracle_matches_reference_on_b200(case):
    # gradient-release goldens come from `_single_param_ranger`, whose Kahan lookahead scales the
    # slow-weight error by alpha (optimi/ranger.py:460); the oracle has that variant behind a flag
    got = run_oracle_case(case, single_param_lookahead=(case.mode == "gr"))
    if case.opt == "stableadamw" and case.dtype == "f32":
        for key, t in got.items():
            assert _rel_close(t, golden_tensor(CUDA, case, key), 1e-6, 1e-9), key
        return
    bad = compare_exact(got, lambda k: golden_tensor(CUDA, case, k), case.name)
    assert not bad, "\n".join(bad)


@pytest.mark.parametrize("case", [c for c in CASES if c.dtype == "f32"], ids=lambda c: c.name)
def test_oracle_matches_reference_on_cpu_f32(case):
    got = run_oracle_case(case, single_param_lookahead=(case.mode == "gr"))
    rtol = 2e-6 if case.opt == "adan" else 1e-6
    for key, t in got.items():
        assert _rel_close(t, golden_tensor(CPU, case, key), rtol, 1e-9), key


def _config1_oracle():
    from cases import CONFIG1_HYPER, config1_grads, config1_params
    from oracle.port import OracleOptimizer

    params = [torch.from_numpy(p) for p in config1_params()]
    opt = OracleOptimizer("adamw", params, **CONFIG1_HYPER)
    for grads in config1_grads():
        opt.step([torch.from_numpy(g) for g in grads])
    return opt


def test_oracle_config1_matches_reference_on_cpu():
    """BASELINE configuration 1 (AdamW float32, 2-layer MLP parameter set, 20 steps) at full size; the
    golden holds every 997th element of what the reference's CPU foreach path produced."""
    from cases import CONFIG1_STRIDE

    opt = _config1_oracle()
    for i, p in enumerate(opt.params):
        for name, t in (("param", p), ("exp_avg", opt.state[i]["exp_avg"]), ("exp_avg_sq", opt.state[i]["exp_avg_sq"])):
            want = torch.from_numpy(CPU[f"config1/{i}.{name}"].copy())
            # parameters that pass close to zero get an absolute floor of 1e-6 of the weights' scale (0.02 .. 0.1)
            atol = 1e-7 if name == "param" else 1e-10
            assert _rel_close(t.reshape(-1)[::CONFIG1_STRIDE], want, 1e-6, atol), f"tensor {i} {name}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("max_norm", [0.05, 1.0, 1e4])
def test_oracle_clip_factor_matches_pytorch_on_cpu(dtype, max_norm):
    """The oracle's restatement of clip_grad_norm_'s coefficient against PyTorch itself (CPU tensors)."""
    from oracle import port

    gen = torch.Generator().manual_seed(11)
    shapes = [(257, 129), (4096,), (1000, 333), (7,), (300, 1024)]
    grads = [(torch.randn(s, generator=gen) * 1e-2).to(dtype) for s in shapes]
    params = []
    for g in grads:
        p = torch.nn.Parameter(torch.zeros_like(g))
        p.grad = g.clone()
        params.append(p)
    total = torch.nn.utils.clip_grad_norm_(params, max_norm)
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    o_coef, o_total = port.clip_factor(grads, max_norm)

    def tol(x):
        # bf16: one unit in the last place.  float32: PyTorch's CPU sum of a few hundred thousand fp32 squares
        # carries a relative error of order 1e-6, the oracle sums in double
        import math

        return 2.0 ** (math.floor(math.log2(abs(x))) - 7) if dtype == torch.bfloat16 else 2e-5 * abs(x)

    assert abs(o_total - float(total)) <= tol(float(total))
    assert abs(o_coef - float(coef)) <= tol(float(coef))
    if o_coef == float(coef):
        for p, g in zip(params, grads):
            assert torch.equal(p.grad, port.scale_gradient(g, o_coef))
