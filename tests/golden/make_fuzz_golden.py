"""Golden outputs of the UNMODIFIED reference for seeded random float32 configurations, on CPU.

Usage (from the repository root):

    python tests/golden/make_fuzz_golden.py --reference <dir holding the optimi package>

Writes ``tests/golden/cpu_fuzz_f32.npz``.  The configurations come from the same generator as the GPU
fuzz test (``tests/test_fuzz_gpu.py: random_config``) with the storage type forced to float32, the
only one for which the reference's CPU path computes what its CUDA path computes; every run uses
``foreach=True, triton=False``.  Inputs are not stored: ``fuzz_inputs(seed)`` regenerates them.
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


def fuzz_inputs(seed: int):
    """(optimizer key, constructor keywords, initial params, per-step gradient lists, per-step learning rates)."""
    from test_fuzz_gpu import random_config

    rng = random.Random(5000 + seed)
    opt, _, kw = random_config(rng)
    kw.pop("kahan_sum", None)  # float32: no Kahan buffers
    g = torch.Generator().manual_seed(5000 + seed)
    shapes = [rng.choice(SHAPES) for _ in range(rng.randint(1, 5))]
    params = [torch.randn(s, generator=g) * rng.choice([0.02, 1.0]) for s in shapes]
    steps = rng.randint(2, 9)
    scale = 10 ** rng.uniform(-5, -1)
    grads = [[torch.zeros(s) if rng.random() < 0.1 else torch.randn(s, generator=g) * scale for s in shapes] for _ in range(steps)]
    lrs = [kw["lr"] * rng.choice([1.0, 0.5, 0.1]) if not kw.get("decouple_lr") else kw["lr"] for _ in range(steps)]
    return opt, kw, params, grads, lrs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="directory that contains the reference's `optimi` package")
    args = ap.parse_args()
    sys.path.insert(0, os.path.abspath(args.reference))
    import optimi

    assert os.path.abspath(optimi.__file__).startswith(os.path.abspath(args.reference)), optimi.__file__
    blob = {}
    for seed in range(N_SEEDS):
        opt, kw, params, grads, lrs = fuzz_inputs(seed)
        ps = [p.clone().requires_grad_(True) for p in params]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            ref = getattr(optimi, CLASS_NAMES[opt])(ps, foreach=True, triton=False, **kw)
        for it, gs in enumerate(grads):
            ref.param_groups[0]["lr"] = lrs[it]
            for p, gr in zip(ps, gs):
                p.grad = gr.clone()
            ref.step()
            ref.zero_grad()
        for i, p in enumerate(ps):
            if p.numel() == 0:
                continue
            blob[f"fuzz{seed}/{i}.param"] = p.detach().numpy().copy()
            for name in STATE_NAMES[opt]:
                t = ref.state[p].get(name)
                if t is not None and t.numel() == p.numel():
                    blob[f"fuzz{seed}/{i}.{name}"] = t.numpy().copy()
    blob["__meta__"] = np.array(f"optimi {optimi.__version__}; torch {torch.__version__}; device cpu; {N_SEEDS} seeds")
    out = os.path.join(HERE, "cpu_fuzz_f32.npz")
    np.savez_compressed(out, **blob)
    print(f"wrote {out}: {len(blob) - 1} arrays, {os.path.getsize(out) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
