"""Pins the CPU oracle against what the unmodified reference computed (CPU, float32, foreach path) for 64
seeded random optimizer / hyper-parameter / learning-rate-schedule combinations — the configurations
the fixed golden cases do not reach (betas of 0 and 0.999, eps down to 1e-10, dampening with
`torch_init`, lookahead every step, zero gradients, one-element tensors)."""

import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
from make_fuzz_golden import N_SEEDS, fuzz_inputs  # noqa: E402

from cases import STATE_NAMES  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "cpu_fuzz_f32.npz"))


@pytest.mark.parametrize("seed", range(N_SEEDS))
def test_oracle_matches_reference_on_random_float32_configurations(seed):
    from oracle.port import OracleOptimizer

    opt, kw, params, grads, lrs = fuzz_inputs(seed)
    oracle = OracleOptimizer(opt, [p.clone() for p in params], **kw)
    for it, gs in enumerate(grads):
        oracle.h["lr"] = lrs[it]
        oracle.step([g.clone() for g in gs])
    checked = 0
    for i, p in enumerate(oracle.params):
        if p.numel() == 0:
            continue
        pairs = [("param", p)]
        for name in STATE_NAMES[opt]:
            t = oracle.state[i].get(name)
            if t is not None and t.numel() == p.numel():
                pairs.append((name, t))
        for name, got in pairs:
            want = torch.from_numpy(GOLDEN[f"fuzz{seed}/{i}.{name}"].copy()).double().reshape(-1)
            got = got.double().reshape(-1)
            # CPU ATen neither fuses multiply-adds nor divides by reciprocals the way CUDA ATen (which the
            # oracle follows) does: 1e-6 relative per op, a few of them chained, over a floor of 1e-6 of the tensor's scale
            tol = 5e-6 * want.abs() + 1e-6 * float(want.abs().max()) + 1e-30
            bad = (got - want).abs() > tol
            assert not bool(bad.any()), f"seed {seed} {opt} {kw} tensor {i} {name}: {int(bad.sum())}/{bad.numel()} off, worst {float(((got - want).abs() / tol).max()):.1f}x"
            checked += 1
    assert checked or all(p.numel() == 0 for p in oracle.params)


CUDA_FUZZ_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "cuda_fuzz.npz")


@pytest.mark.skipif(not os.path.exists(CUDA_FUZZ_PATH), reason="tests/golden/cuda_fuzz.npz has not been generated (make_fuzz_golden.py --device cuda)")
@pytest.mark.parametrize("seed", range(N_SEEDS))
def test_oracle_matches_reference_on_random_configurations_from_a_gpu(seed):
    """Same configurations in their own storage types (bf16 / fp16 / fp32, Kahan as drawn) against what the
    reference's foreach path produced on a CUDA device: bit for bit, StableAdamW at its stated tolerance."""
    from helpers import ulp_diff
    from oracle.port import OracleOptimizer

    golden = np.load(CUDA_FUZZ_PATH)
    opt, kw, params, grads, lrs = fuzz_inputs(seed, float32_only=False)
    oracle = OracleOptimizer(opt, [p.clone() for p in params], **kw)
    for it, gs in enumerate(grads):
        oracle.h["lr"] = lrs[it]
        oracle.step([g.clone() for g in gs])
    for i, p in enumerate(oracle.params):
        if p.numel() == 0:
            continue
        pairs = [("param", p)]
        for name in STATE_NAMES[opt]:
            t = oracle.state[i].get(name)
            if t is not None and t.numel() == p.numel():
                pairs.append((name, t))
        for name, got in pairs:
            raw = golden[f"fuzz{seed}/{i}.{name}"]
            want = torch.from_numpy(raw.copy()) if got.dtype == torch.float32 else torch.from_numpy(raw.view(np.int16).copy()).view(got.dtype)
            got, want = got.reshape(-1), want.reshape(-1)
            where = f"seed {seed} {opt} {kw} tensor {i} {name}"
            if opt == "stableadamw":
                # float16 with a tiny eps: eps^2 underflows to zero, an untouched element then divides 0 by 0, and whole
                # tensors go NaN or infinite in the reference as in the oracle; those must sit at the same places
                same_special = (got.isnan() & want.isnan()) | (got.isinf() & want.isinf() & (got.sign() == want.sign()))
                finite = got.isfinite() & want.isfinite()
                assert bool((same_special | finite).all()), f"{where}: NaN / infinity at different places"
                ok = (got.double() - want.double()).abs() <= 1e-6 + (2e-6 if got.dtype == torch.float32 else 2**-7) * want.double().abs()
                assert bool((ok | same_special).all()), f"{where}: {int((~(ok | same_special)).sum())} elements off"
            else:
                d = ulp_diff(got, want)
                d[got.isnan() & want.isnan()] = 0
                assert int(d.max()) == 0, f"{where}: {int((d > 0).sum())}/{d.numel()} differ, max {int(d.max())} ulp"
