"""Shared helpers of the parity tests: golden loading, bit-level comparison, oracle replays."""

from __future__ import annotations

import os

import numpy as np
import torch

from cases import CASES_BY_NAME, STATE_NAMES, Case, accumulate_on, make_inputs  # noqa: F401

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TORCH_DTYPE = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}

_cache = {}


def load_golden(which: str):
    """which: 'cuda' (reference foreach / per-parameter paths on a B200) or 'cpu_f32'."""
    if which not in _cache:
        _cache[which] = np.load(os.path.join(GOLDEN_DIR, which + ".npz"))
    return _cache[which]


def golden_tensor(blob, case: Case, key: str):
    full = f"{case.name}/{key}"
    if full not in blob.files:
        return None
    arr = blob[full]
    if arr.dtype == np.float32:
        return torch.from_numpy(arr.copy())
    return torch.from_numpy(arr.view(np.int16).copy()).view(TORCH_DTYPE[case.dtype])


def case_tensors(case: Case, device="cpu"):
    """(params, grads[step][i]) in the case's storage dtype, rounded to nearest even from fp32."""
    dt = TORCH_DTYPE[case.dtype]
    p_np, g_np = make_inputs(case)
    params = [torch.from_numpy(p).to(dt).to(device) for p in p_np]
    grads = [[torch.from_numpy(g).to(dt).to(device) for g in gs] for gs in g_np]
    return params, grads


def as_ordered_int(t: torch.Tensor) -> torch.Tensor:
    """Maps floating bit patterns to integers whose difference is the distance in ulps."""
    if t.dtype == torch.float32:
        i = t.contiguous().view(torch.int32).to(torch.int64)
        return torch.where(i < 0, -(i & 0x7FFFFFFF), i)
    i = t.contiguous().view(torch.int16).to(torch.int64)
    return torch.where(i < 0, -(i & 0x7FFF), i)


def ulp_diff(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return (as_ordered_int(a.cpu()) - as_ordered_int(b.cpu())).abs()


def ulp_of(t: torch.Tensor) -> torch.Tensor:
    """Size of one unit in the last place at |t| in t's dtype, as float64 (floored at the smallest normal)."""
    mant = {torch.float32: 23, torch.bfloat16: 7, torch.float16: 10}[t.dtype]
    tiny = {torch.float32: 2.0**-126, torch.bfloat16: 2.0**-126, torch.float16: 2.0**-14}[t.dtype]
    mag = t.abs().double().clamp_min(tiny)
    return torch.pow(2.0, torch.floor(torch.log2(mag)) - mant)


def within_ulps_of_scale(a: torch.Tensor, b: torch.Tensor, n_ulp: float, floor: float) -> torch.Tensor:
    """|a-b| <= n_ulp * ulp(max(|a|,|b|,floor)): the 'within n ulp' test with a magnitude floor, so that
    values straddling zero are not counted as millions of integer steps apart."""
    a, b = a.cpu(), b.cpu()
    scale = torch.maximum(a.abs().double(), b.abs().double()).clamp_min(floor)
    ref = torch.maximum(a.abs(), b.abs()).clamp_min(floor).to(a.dtype)
    return (a.double() - b.double()).abs() <= n_ulp * ulp_of(ref) + 0 * scale


def run_oracle_case(case: Case, single_param_lookahead: bool = False):
    """Replays a golden case through the CPU oracle; returns {key: tensor} in the golden's layout."""
    from oracle.port import OracleOptimizer

    params, grads = case_tensors(case)
    if case.mode == "func":
        fk = dict(case.func_kwargs)
        opt = OracleOptimizer(
            case.opt, params, lr=fk["lr"], betas=(fk["beta1"], fk["beta2"], fk["beta3"]), weight_decay=fk["weight_decay"],
            eps=fk["eps"], adam_wd=fk["adam_wd"], kahan_sum=fk["kahan_sum"],
        )  # fmt: skip
    else:
        kw = dict(case.kwargs)
        opt = OracleOptimizer(case.opt, params, **kw)
    opt.single_param_lookahead = single_param_lookahead
    for it in range(case.steps):
        gs = [g.clone() for g in grads[it]]
        if case.mode == "gr":
            for i, g in enumerate(gs):
                opt.step_param(i, g, accumulate=accumulate_on(it))
        else:
            opt.step(gs)
    out = {}
    for i, p in enumerate(params):
        out[f"{i}.param"] = p
        for name in STATE_NAMES[case.opt]:
            t = opt.state[i].get(name)
            if t is not None:
                out[f"{i}.{name}"] = t
    return out
