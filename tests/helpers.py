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
    ref = torch.maximum(a.abs(), b.abs()).clamp_min(floor).to(a.dtype)
    return (a.double() - b.double()).abs() <= n_ulp * ulp_of(ref)


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


def run_b200_case(case: Case, device="cuda", release_stream: bool = False):
    """Replays a golden case through the optimi_b200 classes (CUDA kernels); same layout as the golden."""
    import warnings

    import optimi_b200
    from cases import CLASS_NAMES

    params, grads = case_tensors(case, device)
    params = [p.requires_grad_(True) for p in params]
    out = {}
    if case.mode == "func":
        g0 = grads[0]
        states = {
            "exp_avg": [torch.zeros_like(p) for p in params],
            "exp_avg_diff": [torch.zeros_like(p) for p in params],
            "exp_avg_sq": [torch.zeros_like(p) for p in params],
            "prev_grad": [g.clone().mul_(-1) for g in g0],
        }
        step = torch.tensor(0, dtype=torch.int32)
        with torch.no_grad():
            for it in range(case.steps):
                optimi_b200.adan(
                    params, [g.clone() for g in grads[it]], states["exp_avg"], states["exp_avg_diff"], states["exp_avg_sq"],
                    states["prev_grad"], None, step=step, **case.func_kwargs,
                )  # fmt: skip
        for i, p in enumerate(params):
            out[f"{i}.param"] = p.detach()
            for name, lst in states.items():
                out[f"{i}.{name}"] = lst[i]
        return out

    cls = getattr(optimi_b200, CLASS_NAMES[case.opt])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = cls(params, **case.kwargs)
    if release_stream:
        opt.use_release_stream(True)
    for it in range(case.steps):
        gs = [g.clone() for g in grads[it]]
        if case.mode == "foreach":
            for p, g in zip(params, gs):
                p.grad = g
            opt.step()
            opt.zero_grad()
        else:
            opt.optimizer_accumulation = accumulate_on(it)
            for p, g in zip(params, gs):
                p.grad = g
                opt.step(param=p)
                opt.zero_grad(param=p)
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        out[f"{i}.param"] = p.detach()
        for name in STATE_NAMES[case.opt]:
            t = opt.state[p].get(name)
            if t is not None and t.numel() == p.numel():
                out[f"{i}.{name}"] = t
    return out


def compare_exact(got: dict, want_of, label: str):
    """Bit-exact comparison of every tensor in `got` against want_of(key); returns a list of failures."""
    bad = []
    for key, t in got.items():
        w = want_of(key)
        if w is None:
            bad.append(f"{label}: no expected tensor for {key}")
            continue
        d = ulp_diff(t.detach().cpu().reshape(-1), w.reshape(-1))
        n = int((d > 0).sum())
        if n:
            bad.append(f"{label}: {key}: {n}/{d.numel()} elements differ, max {int(d.max())} ulp")
    return bad
