"""Python driver of the CPU oracle (TEST INFRASTRUCTURE ONLY — never imported by the product).

`OracleOptimizer` keeps parameters and optimizer states as CPU torch tensors (used purely as typed
storage), computes the per-step host scalars the way the reference's functional entry points do
and calls the C restatement in ``optimi_oracle.c`` once per tensor.  It reproduces what the
reference's classes do around the step as well: lazy state creation with the reference's initial
values, the group-level step counter of whole-list steps and the per-parameter counter of
gradient-release steps.

Reference lines followed:
    host scalars     optimi/adam.py:261-273, lion.py:227-235, sgd.py:256-260, stableadamw.py:327-332,
                     adan.py:290-309, radam.py:262-284, ranger.py:283-305, utils.py:26-36
    state init       optimi/adam.py:95-109, lion.py:89-99, sgd.py:99-121, stableadamw.py:115-135,
                     adan.py:104-120, radam.py:96-110, ranger.py:102-119
"""

from __future__ import annotations

import ctypes
import math
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboptimi_oracle.so")

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


class Scalars(ctypes.Structure):
    _fields_ = [(n, ctypes.c_double) for n in (
        "lr", "beta1_comp", "beta2", "beta2_hat", "beta2_comp", "beta3_hat", "beta3_comp",
        "weight_decay", "eps", "max_lr", "momentum", "rect", "alpha")] + [(n, ctypes.c_int) for n in (
        "decouple_wd", "decouple_lr", "kahan", "update", "dampening", "adam_wd", "lookahead",
        "single_param_lookahead")]  # fmt: skip


def build(force: bool = False) -> str:
    """Compiles the oracle with the Makefile beside this file (gcc, a second or two)."""
    srcs = [os.path.join(_HERE, f) for f in ("optimi_oracle.c", "oracle_ops.inc", "Makefile")]
    if force or not os.path.exists(_LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        assert _lib.oracle_sizeof_scalars() == ctypes.sizeof(Scalars)
    return _lib


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def debias(beta: float, step: int) -> float:
    return 1 - beta**step


def debias_beta(beta: float, step: int) -> float:
    return (beta**step - beta) / (beta**step - 1)


def _rect(beta2: float, step: int) -> float:
    """RAdam's variance rectification term, or -1 while rho <= 5 (the reference's ``None``)."""
    rho_inf = 2 / (1 - beta2) - 1
    rho = rho_inf - 2 * step * (beta2**step) / debias(beta2, step)
    if rho > 5:
        return math.sqrt(((rho - 4) * (rho - 2) * rho_inf) / ((rho_inf - 4) * (rho_inf - 2) * rho))
    return -1.0


DEFAULTS = {
    "adam": dict(betas=(0.9, 0.99), weight_decay=0.0, eps=1e-6, decouple_wd=False, decouple_lr=False, max_lr=None, kahan_sum=None),
    "adamw": dict(betas=(0.9, 0.99), weight_decay=1e-2, eps=1e-6, decouple_wd=True, decouple_lr=False, max_lr=None, kahan_sum=None),
    "lion": dict(betas=(0.9, 0.99), weight_decay=0.0, decouple_lr=False, max_lr=None, kahan_sum=None),
    "sgd": dict(momentum=0.0, weight_decay=0.0, dampening=False, decouple_wd=False, decouple_lr=False, max_lr=None,
                torch_init=False, kahan_sum=None),
    "stableadamw": dict(betas=(0.9, 0.99), weight_decay=1e-2, eps=1e-6, decouple_lr=False, max_lr=None, kahan_sum=None),
    "adan": dict(betas=(0.98, 0.92, 0.99), weight_decay=2e-2, eps=1e-6, decouple_lr=False, max_lr=None, adam_wd=False,
                 kahan_sum=False),
    "radam": dict(betas=(0.9, 0.99), weight_decay=0.0, eps=1e-6, decouple_wd=False, decouple_lr=False, max_lr=None,
                  kahan_sum=None),
    "ranger": dict(betas=(0.9, 0.99), weight_decay=0.0, eps=1e-6, k=6, alpha=0.5, decouple_wd=True, decouple_lr=False,
                   max_lr=None, kahan_sum=None),
}  # fmt: skip


class OracleOptimizer:
    """One parameter group of one reference optimizer, stepped on the CPU through the C oracle."""

    def __init__(self, opt: str, params: list[torch.Tensor], lr: float, **kw):
        kw.pop("gradient_release", None)
        kw.pop("foreach", None)
        kw.pop("triton", None)
        h = dict(DEFAULTS[opt])
        unknown = set(kw) - set(h)
        assert not unknown, unknown
        h.update(kw)
        h["lr"] = lr
        if h.get("decouple_lr") and h.get("max_lr") is None:
            h["max_lr"] = lr  # optimi/optimizer.py:20-21
        self.opt, self.h, self.params = opt, h, params
        self.state: list[dict] = [dict() for _ in params]
        self.group_step = 0
        self.single_param_lookahead = False  # set True to follow optimi/ranger.py:455-465 in step_param

    # ------------------------------------------------------------------ state
    def _init_state(self, i: int, grad: torch.Tensor):
        st, p, h = self.state[i], self.params[i], self.h
        if st:
            return
        low = p.dtype in (torch.float16, torch.bfloat16)
        st["kahan_comp"] = torch.zeros_like(p) if (h["kahan_sum"] or h["kahan_sum"] is None) and low else None
        st["step"] = 0
        o = self.opt
        if o in ("adam", "adamw", "radam", "ranger", "stableadamw"):
            st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
        if o == "ranger":
            st["la_param"] = p.clone()
        if o == "lion":
            st["exp_avg"] = torch.zeros_like(p)
        if o == "sgd":
            if h["dampening"] and h["torch_init"]:
                st["exp_avg"] = grad.clone()
                if h["weight_decay"] != 0 and not h["decouple_lr"] and not h["decouple_wd"]:
                    # Tensor.add_(param, alpha=wd): one fused multiply-add, rounded once
                    st["exp_avg"] = _fma_round(grad, p, h["weight_decay"])
            elif h["momentum"] != 0:
                st["exp_avg"] = torch.zeros_like(p)
            else:
                st["exp_avg"] = None
        if o == "adan":
            st["exp_avg"], st["exp_avg_diff"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p), torch.zeros_like(p)
            st["prev_grad"] = grad.clone().mul_(-1)
        if o == "stableadamw":
            st["eps_sq"] = torch.tensor(h["eps"] ** 2, dtype=p.dtype)

    # ---------------------------------------------------------------- scalars
    def _scalars(self, step: int, update: bool) -> Scalars:
        h, o = self.h, self.opt
        s = Scalars()
        s.lr, s.update = h["lr"], int(update)
        s.max_lr = h["max_lr"] if h.get("max_lr") is not None else 0.0
        s.decouple_lr = int(bool(h.get("decouple_lr")))
        s.rect, s.alpha = -1.0, 0.0
        wd = h["weight_decay"]
        if o in ("adam", "adamw", "radam", "ranger", "stableadamw"):
            b1, b2 = h["betas"]
            s.beta1_comp = 1 - debias_beta(b1, step)
            s.beta2_hat = debias_beta(b2, step)
            s.beta2_comp = 1 - s.beta2_hat
            s.eps = h["eps"]
        if o in ("adam", "adamw", "radam", "ranger", "sgd"):
            if wd != 0:
                if h["decouple_lr"]:
                    wd = 1 - (h["lr"] / h["max_lr"]) * wd
                elif h["decouple_wd"]:
                    wd = 1 - h["lr"] * wd
            s.decouple_wd = int(bool(h["decouple_wd"] or h["decouple_lr"]))
        if o in ("radam", "ranger"):
            s.rect = _rect(h["betas"][1], step)
        if o == "ranger":
            s.alpha = h["alpha"]
            s.lookahead = int(step % h["k"] == 0)
            s.single_param_lookahead = int(self.single_param_lookahead)
        if o == "lion":
            b1, b2 = h["betas"]
            s.beta1_comp, s.beta2_comp = 1 - b1, 1 - b2
            if wd != 0:
                wd = 1 - (h["lr"] / h["max_lr"]) * wd if h["decouple_lr"] else 1 - h["lr"] * wd
        if o == "sgd":
            s.momentum, s.dampening = h["momentum"], int(bool(h["dampening"]))
        if o == "adan":
            b1, b2, b3 = h["betas"]
            s.beta1_comp = 1 - debias_beta(b1, step)
            s.beta2 = b2
            s.beta2_comp = 1 - debias_beta(b2, step)
            s.beta3_hat = debias_beta(b3, step)
            s.beta3_comp = 1 - s.beta3_hat
            s.eps = h["eps"]
            s.adam_wd = int(bool(h["adam_wd"]))
            if wd != 0:
                wd = (h["lr"] / h["max_lr"]) * wd if h["decouple_lr"] else h["lr"] * wd
                wd = 1 - wd if h["adam_wd"] else 1 + wd
        s.weight_decay = wd
        return s

    # ------------------------------------------------------------------ steps
    def _apply(self, i: int, grad: torch.Tensor, s: Scalars):
        p, st, L = self.params[i], self.state[i], lib()
        n, dt = p.numel(), DTYPE_CODE[p.dtype]
        k = st["kahan_comp"]
        s.kahan = int(k is not None)
        o = self.opt
        if o in ("adam", "adamw"):
            rc = L.oracle_adam(_ptr(p), _ptr(grad), _ptr(st["exp_avg"]), _ptr(st["exp_avg_sq"]), _ptr(k), ctypes.c_int64(n), dt, ctypes.byref(s))
        elif o == "lion":
            rc = L.oracle_lion(_ptr(p), _ptr(grad), _ptr(st["exp_avg"]), _ptr(k), ctypes.c_int64(n), dt, ctypes.byref(s))
        elif o == "sgd":
            rc = L.oracle_sgd(_ptr(p), _ptr(grad), _ptr(st["exp_avg"]), _ptr(k), ctypes.c_int64(n), dt, ctypes.byref(s))
        elif o == "stableadamw":
            e = st["eps_sq"]
            bits = e.view(torch.int32).item() & 0xFFFFFFFF if e.dtype == torch.float32 else e.view(torch.int16).item() & 0xFFFF
            rc = L.oracle_stableadamw(_ptr(p), _ptr(grad), _ptr(st["exp_avg"]), _ptr(st["exp_avg_sq"]), _ptr(k), ctypes.c_int64(n), dt,
                                      ctypes.c_uint32(bits), ctypes.byref(s))  # fmt: skip
        elif o == "adan":
            rc = L.oracle_adan(_ptr(p), _ptr(grad), _ptr(st["exp_avg"]), _ptr(st["exp_avg_diff"]), _ptr(st["exp_avg_sq"]),
                               _ptr(st["prev_grad"]), _ptr(k), ctypes.c_int64(n), dt, ctypes.byref(s))  # fmt: skip
        else:
            rc = L.oracle_radam_ranger(_ptr(p), _ptr(grad), _ptr(st["exp_avg"]), _ptr(st["exp_avg_sq"]), _ptr(st.get("la_param")),
                                       _ptr(k), ctypes.c_int64(n), dt, ctypes.byref(s))  # fmt: skip
        assert rc == 0

    def step(self, grads: list[torch.Tensor]):
        """Whole-list step with a group-level counter (the reference's ``step()`` without ``param``)."""
        for i, g in enumerate(grads):
            self._init_state(i, g)
        self.group_step += 1
        for i, g in enumerate(grads):
            self._apply(i, g, self._scalars(self.group_step, True))

    def step_param(self, i: int, grad: torch.Tensor, accumulate: bool = False):
        """Per-parameter step with a per-parameter counter (the reference's ``step(param=p)``); the
        counter advances on accumulation micro-steps too (optimi/adam.py:261)."""
        self._init_state(i, grad)
        self.state[i]["step"] += 1
        self._apply(i, grad, self._scalars(self.state[i]["step"], not accumulate))


def _fma_round(g: torch.Tensor, p: torch.Tensor, alpha: float) -> torch.Tensor:
    """round_to_dtype(fma(fp32(alpha), p, g)) — ``g.add_(p, alpha=alpha)`` as one fused op."""
    a = float(torch.tensor(alpha, dtype=torch.float32))
    return (g.double() + a * p.double()).float().to(g.dtype)


# ------------------------------------------------------------------------------------------------
# Gradient scaling next to the step.  These restate PyTorch, not the reference (which leaves
# clipping and loss-scale unscaling to its callers): torch/nn/utils/clip_grad.py `_get_total_norm`
# and `_clip_grads_with_norm_`, and the arithmetic of `torch._foreach_mul_(grads, scalar_tensor)`.
# ------------------------------------------------------------------------------------------------
def scale_gradient(grad: torch.Tensor, factor: float) -> torch.Tensor:
    """`grad * factor` as `_foreach_mul_` with a 0-dim tensor computes it: fp32 product of the element and
    the fp32 factor, one rounding to the gradient's dtype."""
    f = torch.tensor(factor, dtype=torch.float32)
    return (grad.float() * f).to(grad.dtype)


def clip_factor(grads: list[torch.Tensor], max_norm: float) -> tuple[float, float]:
    """(coefficient, total norm) of `torch.nn.utils.clip_grad_norm_(params, max_norm)` for gradients of one dtype,
    every intermediate rounded to that dtype as PyTorch's tensor arithmetic rounds it:

        norms  = [round(sqrt(sum g^2)) for g in grads]            torch._foreach_norm
        total  = round(sqrt(sum norms^2))                          torch.linalg.vector_norm(torch.stack(norms))
        coef   = round(round(1 / round(total + 1e-6)) * max_norm)  Tensor.__rtruediv__ is reciprocal() * other
        coef   = min(coef, 1)                                      torch.clamp(max=1.0), NaN kept

    Sums of squares are taken in double here, so results can differ from PyTorch's fp32 sums by one unit of
    the dtype."""
    dtype = grads[0].dtype

    def rnd(x: float) -> float:
        return float(torch.tensor(x, dtype=torch.float32).to(dtype))

    def f32(x: float) -> float:
        return float(torch.tensor(x, dtype=torch.float32))

    norms = [rnd(f32(math.sqrt(f32(float(g.double().square().sum()))))) for g in grads]
    total = rnd(f32(math.sqrt(f32(sum(n * n for n in norms)))))
    denom = rnd(f32(total + f32(1e-6)))
    recip = rnd(f32(1.0 / denom)) if denom != 0 else float("inf")
    coef = rnd(f32(recip * f32(max_norm)))
    if coef > 1.0:
        coef = 1.0
    return coef, total
