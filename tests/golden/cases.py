"""Golden-vector case table and seeded input generator for the optimizer-step parity tests.

Every case names one optimizer, its constructor keywords, a storage dtype, a run mode and a step
count.  Inputs come from numpy's PCG64 stream (stable for a given seed), so the script that makes
the golden outputs and the tests that replay the same case see bit-identical parameters and
gradients without the inputs being stored.

Run modes
    "foreach"  whole-list step per iteration, the reference's ``_foreach_*`` functions
               (e.g. optimi/adam.py:399-453).
    "gr"       one ``step(param=p)`` per parameter per iteration, the reference's gradient-release
               route through ``_single_param_*`` (e.g. optimi/adam.py:183-208, 354-396), with
               optimizer accumulation switched on for three of every four iterations
               (optimi/optimizer.py:74-82).
    "func"     the functional entry point called directly (only used for Adan's ``adam_wd`` flag,
               which the class never forwards: optimi/adan.py:181-203).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

# (shape, initialiser): a 2-D weight, a norm weight of ones, a 1-D normal vector, a zero bias.
# Odd element counts exercise the scalar tail of the vectorised kernels.
SHAPES = [((31, 33), "normal"), ((129,), "ones"), ((512,), "normal"), ((7,), "zeros")]

# names of the per-parameter state tensors each optimizer keeps, in the order of the reference's
# functional signatures (optimi/adam.py:213-218, lion.py:187-191, sgd.py:214-218,
# stableadamw.py:277-283, adan.py:236-243, radam.py:214-219, ranger.py:229-235)
STATE_NAMES = {
    "adam": ["exp_avg", "exp_avg_sq", "kahan_comp"],
    "adamw": ["exp_avg", "exp_avg_sq", "kahan_comp"],
    "lion": ["exp_avg", "kahan_comp"],
    "sgd": ["exp_avg", "kahan_comp"],
    "stableadamw": ["exp_avg", "exp_avg_sq", "kahan_comp"],
    "adan": ["exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp"],
    "radam": ["exp_avg", "exp_avg_sq", "kahan_comp"],
    "ranger": ["exp_avg", "exp_avg_sq", "la_param", "kahan_comp"],
}

CLASS_NAMES = {
    "adam": "Adam", "adamw": "AdamW", "lion": "Lion", "sgd": "SGD", "stableadamw": "StableAdamW",
    "adan": "Adan", "radam": "RAdam", "ranger": "Ranger",
}  # fmt: skip


@dataclass
class Case:
    name: str
    opt: str
    kwargs: dict
    dtype: str  # "f32" | "bf16" | "f16"
    mode: str = "foreach"
    steps: int = 12
    seed: int = 0
    func_kwargs: dict = field(default_factory=dict)  # mode "func" only


def _dtype_variants():
    # (tag, storage dtype, kahan_sum keyword)
    return [("f32", "f32", None), ("bf16k", "bf16", None), ("bf16n", "bf16", False), ("f16k", "f16", None)]


def build_cases() -> list[Case]:
    cases: list[Case] = []
    seed = 100

    def add(name, opt, kwargs, dtype, **kw):
        nonlocal seed
        seed += 1
        cases.append(Case(name=name, opt=opt, kwargs=dict(kwargs), dtype=dtype, seed=seed, **kw))

    lr = 3e-4
    wd_modes_adam = {
        "nowd": dict(weight_decay=0.0),
        "l2": dict(weight_decay=1e-2),
        "dwd": dict(weight_decay=1e-2, decouple_wd=True),
        "dlr": dict(weight_decay=1e-5, decouple_lr=True),
    }
    for tag, dt, ks in _dtype_variants():
        for wtag, wkw in wd_modes_adam.items():
            add(f"adam_{tag}_{wtag}", "adam", dict(lr=lr, kahan_sum=ks, **wkw), dt)
            add(f"radam_{tag}_{wtag}", "radam", dict(lr=lr, kahan_sum=ks, **wkw), dt)
        # Ranger defaults to decouple_wd=True (optimi/ranger.py:68)
        add(f"ranger_{tag}_nowd", "ranger", dict(lr=lr, kahan_sum=ks), dt)
        add(f"ranger_{tag}_dwd", "ranger", dict(lr=lr, kahan_sum=ks, weight_decay=1e-2), dt)
        add(f"ranger_{tag}_l2", "ranger", dict(lr=lr, kahan_sum=ks, weight_decay=1e-2, decouple_wd=False), dt)
        add(f"ranger_{tag}_dlr", "ranger", dict(lr=lr, kahan_sum=ks, weight_decay=1e-5, decouple_lr=True, k=4, alpha=0.8), dt)

        add(f"adamw_{tag}_default", "adamw", dict(lr=lr, kahan_sum=ks), dt)
        add(f"adamw_{tag}_dlr", "adamw", dict(lr=lr, kahan_sum=ks, weight_decay=1e-5, decouple_lr=True), dt)

        for wtag, wkw in {
            "nowd": dict(weight_decay=0.0),
            "dwd": dict(weight_decay=1e-1),
            "dlr": dict(weight_decay=1e-5, decouple_lr=True),
        }.items():
            add(f"lion_{tag}_{wtag}", "lion", dict(lr=1e-4, kahan_sum=ks, **wkw), dt)
            add(f"stableadamw_{tag}_{wtag}", "stableadamw", dict(lr=lr, kahan_sum=ks, **wkw), dt)

        # Adan's kahan_sum default is False, not None (optimi/adan.py:72)
        adan_ks = False if ks is False else (True if dt != "f32" else False)
        for wtag, wkw in {
            "nowd": dict(weight_decay=0.0),
            "wd": dict(weight_decay=2e-2),
            "dlr": dict(weight_decay=1e-5, decouple_lr=True),
        }.items():
            add(f"adan_{tag}_{wtag}", "adan", dict(lr=lr, kahan_sum=adan_ks, **wkw), dt)

        sgd_variants = {
            "plain_l2": dict(momentum=0.0, weight_decay=1e-2),
            "mom_nowd": dict(momentum=0.9),
            "mom_l2": dict(momentum=0.9, weight_decay=1e-2),
            "mom_dwd": dict(momentum=0.9, weight_decay=1e-2, decouple_wd=True),
            "mom_dlr": dict(momentum=0.9, weight_decay=1e-5, decouple_lr=True),
            "damp_l2": dict(momentum=0.9, dampening=True, weight_decay=1e-2),
            "damp_tinit_l2": dict(momentum=0.9, dampening=True, torch_init=True, weight_decay=1e-2),
            "plain_dwd": dict(momentum=0.0, weight_decay=1e-2, decouple_wd=True),
        }
        for stag, skw in sgd_variants.items():
            add(f"sgd_{tag}_{stag}", "sgd", dict(lr=1e-2, kahan_sum=ks, **skw), dt)

    # gradient release + optimizer accumulation (per-parameter steps)
    for tag, dt in [("f32", "f32"), ("bf16k", "bf16")]:
        gr = dict(gradient_release=True)
        add(f"gr_adam_{tag}_dwd", "adam", dict(lr=lr, weight_decay=1e-2, decouple_wd=True, **gr), dt, mode="gr", steps=16)
        add(f"gr_adam_{tag}_l2", "adam", dict(lr=lr, weight_decay=1e-2, **gr), dt, mode="gr", steps=16)
        add(f"gr_lion_{tag}_dwd", "lion", dict(lr=1e-4, weight_decay=1e-1, **gr), dt, mode="gr", steps=16)
        add(f"gr_sgd_{tag}_mom_l2", "sgd", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2, **gr), dt, mode="gr", steps=16)
        add(f"gr_stableadamw_{tag}_dwd", "stableadamw", dict(lr=lr, **gr), dt, mode="gr", steps=16)
        add(f"gr_adan_{tag}_wd", "adan", dict(lr=lr, kahan_sum=(dt != "f32"), **gr), dt, mode="gr", steps=16)
        add(f"gr_radam_{tag}_dwd", "radam", dict(lr=lr, weight_decay=1e-2, decouple_wd=True, **gr), dt, mode="gr", steps=16)
        add(f"gr_ranger_{tag}_dwd", "ranger", dict(lr=lr, weight_decay=1e-2, k=4, **gr), dt, mode="gr", steps=16)

    # Adan with Adam-style weight decay: only reachable through the functional API
    for tag, dt in [("f32", "f32"), ("bf16n", "bf16")]:
        add(
            f"func_adan_{tag}_adamwd", "adan", dict(), dt, mode="func",
            func_kwargs=dict(lr=lr, beta1=0.98, beta2=0.92, beta3=0.99, weight_decay=2e-2, eps=1e-6,
                             adam_wd=True, kahan_sum=False),
        )  # fmt: skip
    return cases


CASES = build_cases()
CASES_BY_NAME = {c.name: c for c in CASES}


def make_inputs(case: Case):
    """Returns (params, grads) as float32 numpy arrays: ``params[i]`` and ``grads[step][i]``.

    Weights ~N(0, 0.02^2), norm weights 1, biases 0; gradients ~N(0,1) times a per-tensor
    log-normal scale (median 1e-3, sigma 1), the distribution the benchmark configurations use.
    Callers cast to the case's storage dtype with round-to-nearest-even.
    """
    rng = np.random.default_rng(case.seed)
    params = []
    for shape, init in SHAPES:
        if init == "normal":
            params.append((rng.standard_normal(shape) * 0.02).astype(np.float32))
        elif init == "ones":
            params.append(np.ones(shape, dtype=np.float32))
        else:
            params.append(np.zeros(shape, dtype=np.float32))
    scales = np.exp(rng.normal(np.log(1e-3), 1.0, size=len(SHAPES)))
    grads = []
    for _ in range(case.steps):
        grads.append([(rng.standard_normal(shape) * scales[i]).astype(np.float32) for i, (shape, _) in enumerate(SHAPES)])
    return params, grads


def accumulate_on(step_index: int) -> bool:
    """Gradient-release cases: iterations 0,1,2 of every four only accumulate into the states."""
    return step_index % 4 != 3


# ------------------------------------------------------------------------------------------------
# BASELINE configuration 1: AdamW float32 on the parameters of a 2-layer MLP (Linear 1024->4096 + bias,
# Linear 4096->1024 + bias, 8 393 728 parameters), weights ~N(0, 0.02^2), biases 0, fresh gradients
# ~N(0, (1e-3)^2) every step from seed 0, lr 1e-3, betas (0.9, 0.99), eps 1e-6, weight decay 1e-2 (decoupled),
# 20 steps.  Too large to store: the golden keeps every 997th element of each result tensor.
# ------------------------------------------------------------------------------------------------
CONFIG1_SHAPES = [(4096, 1024), (4096,), (1024, 4096), (1024,)]
CONFIG1_HYPER = dict(lr=1e-3, betas=(0.9, 0.99), eps=1e-6, weight_decay=1e-2, decouple_lr=False)
CONFIG1_STEPS = 20
CONFIG1_STRIDE = 997


def config1_params():
    rng = np.random.default_rng(0)
    return [(rng.standard_normal(s) * 0.02).astype(np.float32) if len(s) == 2 else np.zeros(s, dtype=np.float32) for s in CONFIG1_SHAPES]


def config1_grads():
    """Generator of per-step gradient lists (float32 numpy), seed 0."""
    rng = np.random.default_rng(0)
    for _ in range(CONFIG1_STEPS):
        yield [(rng.standard_normal(s) * 1e-3).astype(np.float32) for s in CONFIG1_SHAPES]
