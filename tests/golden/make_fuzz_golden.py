"""Golden outputs of the UNMODIFIED reference for seeded random configurations.

Usage (from the repository root):

    python tests/golden/make_fuzz_golden.py --reference <dir holding the optimi package>                 # CPU
    python tests/golden/make_fuzz_golden.py --reference <dir holding the optimi package> --device cuda   # on a GPU

``--device cpu`` writes ``tests/golden/cpu_fuzz_f32.npz``: the configurations of the GPU fuzz test's generator
(``tests/test_fuzz_gpu.py: random_config``) with the storage type forced to float32, the only one for which
the reference's CPU path computes what its CUDA path computes.  ``--device cuda`` writes
``tests/golden/cuda_fuzz.npz`` with the generator's own storage types (float32, bfloat16, float16, Kahan
buffers as drawn), arrays as raw bit patterns.  Every run uses ``foreach=True, triton=False``.  Inputs are
not stored: ``fuzz_inputs(seed, ...)`` regenerates them.
"""

from __future__ import annotations

import argparse
import os
import random
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
from cases import CLASS_NAMES, STATE_NAMES  # noqa: E402

N_SEEDS = 64
SHAPES = [(0,), (1,), (7,), (333,), (1024,), (33, 31)]


TORCH_DTYPE = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def fuzz_inputs(seed: int, float32_only: bool = True):
    """(optimizer key, constructor keywords, initial params, per-step gradient lists, per-step learning rates);
    tensors in the storage type drawn for the seed, or float32 when `float32_only`."""
    from test_fuzz_gpu import random_config

    rng = random.Random(5000 + seed)
    opt, dt, kw = random_config(rng)
    if float32_only:
        dt = "f32"
        kw.pop("kahan_sum", None)  # float32: no Kahan buffers
    dtype = TORCH_DTYPE[dt]
    g = torch.Generator().manual_seed(5000 + seed)
    shapes = [rng.choice(SHAPES) for _ in range(rng.randint(1, 5))]
    params = [(torch.randn(s, generator=g) * rng.choice([0.02, 1.0])).to(dtype) for s in shapes]
    steps = rng.randint(2, 9)
    scale = 10 ** rng.uniform(-5, -1)
    grads = [[(torch.zeros(s) if rng.random() < 0.1 else torch.randn(s, generator=g) * scale).to(dtype) for s in shapes] for _ in range(steps)]
    lrs = [kw["lr"] * rng.choice([1.0, 0.5, 0.1]) if not kw.get("decouple_lr") else kw["lr"] for _ in range(steps)]
    return opt, kw, params, grads, lrs


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return t.numpy().copy()
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory that contains the reference's `optimi` package")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    args = ap.parse_args()
    sys.path.insert(0, os.path.abspath(args.reference))
    import optimi

    assert os.path.abspath(optimi.__file__).startswith(os.path.abspath(args.reference)), optimi.__file__
    blob = {}
    for seed in range(N_SEEDS):
        opt, kw, params, grads, lrs = fuzz_inputs(seed, float32_only=args.device == "cpu")
        ps = [p.clone().to(args.device).requires_grad_(True) for p in params]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            ref = getattr(optimi, CLASS_NAMES[opt])(ps, foreach=True, triton=False, **kw)
        for it, gs in enumerate(grads):
            ref.param_groups[0]["lr"] = lrs[it]
            for p, gr in zip(ps, gs):
                p.grad = gr.clone().to(args.device)
            ref.step()
            ref.zero_grad()
        for i, p in enumerate(ps):
            if p.numel() == 0:
                continue
            blob[f"fuzz{seed}/{i}.param"] = to_bits(p)
            for name in STATE_NAMES[opt]:
                t = ref.state[p].get(name)
                if t is not None and t.numel() == p.numel():
                    blob[f"fuzz{seed}/{i}.{name}"] = to_bits(t)
    blob["__meta__"] = np.array(f"optimi {optimi.__version__}; torch {torch.__version__}; device {args.device}; {N_SEEDS} seeds")
    out = os.path.join(HERE, "cpu_fuzz_f32.npz" if args.device == "cpu" else "cuda_fuzz.npz")
    np.savez_compressed(out, **blob)
    print(f"wrote {out}: {len(blob) - 1} arrays, {os.path.getsize(out) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
