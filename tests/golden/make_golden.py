"""Generates golden outputs by running the UNMODIFIED reference optimizers on the seeded cases.

Usage (from the repository root):

    python tests/golden/make_golden.py --reference <dir holding the optimi package> --device cpu
    python tests/golden/make_golden.py --reference <dir holding the optimi package> --device cuda

``--device cpu`` writes ``tests/golden/cpu_f32.npz`` (float32 cases only: CPU ATen rounds in-place
Python scalars to the tensor dtype for bf16/fp16, so its low-precision results are not what the CUDA
foreach functors produce).  ``--device cuda`` writes ``tests/golden/cuda.npz`` with every case; the
committed file was produced on a B200 with torch 2.11.0+cu128.

Every run uses ``foreach=True, triton=False`` (whole-list cases) or ``foreach=False, triton=False``
(gradient-release cases), i.e. the reference's ATen paths and never its Triton kernels.
Arrays are stored as raw bit patterns: float32 as is, bf16/fp16 as uint16.
"""

from __future__ import annotations

import argparse
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, CLASS_NAMES, STATE_NAMES, accumulate_on, make_inputs  # noqa: E402

TORCH_DTYPE = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return t.numpy().copy()
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def run_case(optimi, case, device):
    dtype = TORCH_DTYPE[case.dtype]
    params_np, grads_np = make_inputs(case)
    params = [torch.from_numpy(p).to(dtype).to(device).requires_grad_(True) for p in params_np]
    out = {}

    def grads_for(it):
        return [torch.from_numpy(g).to(dtype).to(device) for g in grads_np[it]]

    if case.mode == "func":
        # functional API with hand-made states (Adan: optimi/adan.py:104-109 initial values)
        g0 = grads_for(0)
        states = {
            "exp_avg": [torch.zeros_like(p) for p in params],
            "exp_avg_diff": [torch.zeros_like(p) for p in params],
            "exp_avg_sq": [torch.zeros_like(p) for p in params],
            "prev_grad": [g.clone().mul_(-1) for g in g0],
        }
        step = torch.tensor(0, dtype=torch.int32)
        with torch.no_grad():
            for it in range(case.steps):
                optimi.adan(
                    [p for p in params], grads_for(it), states["exp_avg"], states["exp_avg_diff"], states["exp_avg_sq"],
                    states["prev_grad"], None, step=step, foreach=True, triton=False, **case.func_kwargs,
                )  # fmt: skip
        for i, p in enumerate(params):
            out[f"{i}.param"] = to_bits(p)
            for name, lst in states.items():
                out[f"{i}.{name}"] = to_bits(lst[i])
        return out

    cls = getattr(optimi, CLASS_NAMES[case.opt])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        if case.mode == "foreach":
            opt = cls(params, foreach=True, triton=False, **case.kwargs)
        else:
            opt = cls(params, foreach=False, triton=False, **case.kwargs)

    for it in range(case.steps):
        grads = grads_for(it)
        if case.mode == "foreach":
            for p, g in zip(params, grads):
                p.grad = g
            opt.step()
            opt.zero_grad()
        else:
            opt.optimizer_accumulation = accumulate_on(it)
            for p, g in zip(params, grads):
                p.grad = g
                opt.step(param=p)
                opt.zero_grad(param=p)

    for i, p in enumerate(params):
        out[f"{i}.param"] = to_bits(p)
        st = opt.state[p]
        for name in STATE_NAMES[case.opt]:
            if st.get(name) is not None and st[name].numel() == p.numel():
                out[f"{i}.{name}"] = to_bits(st[name])
    return out


def run_config1(optimi, device):
    """BASELINE configuration 1 through the reference's foreach path; returns strided samples."""
    from cases import CONFIG1_HYPER, CONFIG1_STRIDE, config1_grads, config1_params

    params = [torch.from_numpy(p).to(device).requires_grad_(True) for p in config1_params()]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = optimi.AdamW(params, foreach=True, triton=False, **CONFIG1_HYPER)
    for grads in config1_grads():
        for p, g in zip(params, grads):
            p.grad = torch.from_numpy(g).to(device)
        opt.step()
        opt.zero_grad()
    out = {}
    for i, p in enumerate(params):
        out[f"{i}.param"] = to_bits(p.detach().reshape(-1)[::CONFIG1_STRIDE])
        for name in ("exp_avg", "exp_avg_sq"):
            out[f"{i}.{name}"] = to_bits(opt.state[p][name].reshape(-1)[::CONFIG1_STRIDE])
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory that contains the reference's `optimi` package")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    sys.path.insert(0, os.path.abspath(args.reference))
    import optimi

    assert os.path.abspath(optimi.__file__).startswith(os.path.abspath(args.reference)), optimi.__file__

    blob = {}
    n = 0
    for case in CASES:
        if args.device == "cpu" and case.dtype != "f32":
            continue
        res = run_case(optimi, case, args.device)
        for k, v in res.items():
            blob[f"{case.name}/{k}"] = v
        n += 1
    for k, v in run_config1(optimi, args.device).items():
        blob[f"config1/{k}"] = v
    blob["__meta__"] = np.array(
        f"optimi {optimi.__version__}; torch {torch.__version__}; device {args.device}"
        + (f" ({torch.cuda.get_device_name(0)})" if args.device == "cuda" else "")
    )
    out = args.out or os.path.join(HERE, "cuda.npz" if args.device == "cuda" else "cpu_f32.npz")
    np.savez_compressed(out, **blob)
    print(f"wrote {out}: {n} cases, {len(blob) - 1} arrays, {os.path.getsize(out) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
