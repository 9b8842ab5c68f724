"""Host scalar arithmetic of every optimizer: the values that follow `dtype` in the C signatures.

One function per optimizer turns the hyper-parameters of a parameter group and the step count `t`
into the tuple of doubles and flags its C entry point expects.  The arithmetic is the reference's,
in Python doubles and in the reference's order of operations (optimi/adam.py:261-273,
lion.py:227-235, sgd.py:256-260, stableadamw.py:327-332, adan.py:290-309, radam.py:262-284,
ranger.py:283-305, utils.py:26-36), so the fp32 values the kernels narrow them to are the ones the
reference's ATen ops receive.  Both the functional API and the per-parameter fast path of gradient
release call these.
"""

from __future__ import annotations

import math


def debias(beta: float, step: int) -> float:
    """Adam's bias-correction denominator 1 - beta^step (optimi/utils.py:26-28)."""
    return 1 - beta**step


def debias_beta(beta: float, step: int) -> float:
    """Beta with the bias correction folded in, beta*(1-beta^(step-1))/(1-beta^step) in the
    reference's simplified form (optimi/utils.py:31-36); 0 at step 1."""
    return (beta**step - beta) / (beta**step - 1)


def fold_weight_decay(weight_decay: float, lr: float, decouple_wd: bool, decouple_lr: bool, max_lr: float | None) -> float:
    """The multiplicative factor for (fully) decoupled decay, or the raw L2 coefficient."""
    if weight_decay != 0:
        if decouple_lr:
            return 1 - (lr / max_lr) * weight_decay
        if decouple_wd:
            return 1 - lr * weight_decay
    return weight_decay


def rectification(beta2: float, step: int) -> float | None:
    """RAdam's variance rectification term; None while the SMA length is at most 5."""
    rho_inf = 2 / (1 - beta2) - 1
    rho = rho_inf - 2 * step * (beta2**step) / debias(beta2, step)
    if rho > 5:
        return math.sqrt(((rho - 4) * (rho - 2) * rho_inf) / ((rho_inf - 4) * (rho_inf - 2) * rho))
    return None


def adam_tail(t, update, *, lr, beta1, beta2, weight_decay, eps, decouple_wd, decouple_lr=False, max_lr=None, kahan_sum=False):
    beta2_hat = debias_beta(beta2, t)
    wd = fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    return (lr, 1 - debias_beta(beta1, t), beta2_hat, 1 - beta2_hat, wd, eps, int(decouple_wd or decouple_lr),
            int(bool(kahan_sum)), int(update))  # fmt: skip


def lion_tail(t, update, *, lr, beta1, beta2, weight_decay, decouple_lr=False, max_lr=None, kahan_sum=False):
    wd = fold_weight_decay(weight_decay, lr, True, decouple_lr, max_lr)  # always decoupled
    return (lr, 1 - beta1, 1 - beta2, wd, int(bool(kahan_sum)), int(update))


def sgd_tail(t, update, *, lr, momentum, weight_decay, dampening, decouple_wd, decouple_lr=False, max_lr=None, kahan_sum=False):
    wd = fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    return (lr, momentum, wd, int(bool(dampening)), int(decouple_wd or decouple_lr), int(bool(kahan_sum)), int(update))


def stableadamw_tail(t, update, *, lr, beta1, beta2, weight_decay, eps, decouple_lr=False, max_lr=None, kahan_sum=False):
    """Everything up to (not including) the workspace pointer and size.  The weight decay stays raw:
    its factor depends on the clipped learning rate, which only the device knows."""
    beta2_hat = debias_beta(beta2, t)
    return (lr, 1 - debias_beta(beta1, t), beta2_hat, 1 - beta2_hat, weight_decay, eps, int(bool(decouple_lr)),
            float(max_lr) if max_lr is not None else 0.0, int(bool(kahan_sum)), int(update))  # fmt: skip


def adan_tail(t, update, *, lr, beta1, beta2, beta3, weight_decay, eps, decouple_lr=False, max_lr=None, adam_wd=False,
              kahan_sum=False):  # fmt: skip
    beta3_hat = debias_beta(beta3, t)
    wd = weight_decay
    if wd != 0:
        wd = (lr / max_lr) * wd if decouple_lr else lr * wd
        wd = 1 - wd if adam_wd else 1 + wd
    return (lr, 1 - debias_beta(beta1, t), beta2, 1 - debias_beta(beta2, t), beta3_hat, 1 - beta3_hat, eps, wd,
            int(bool(adam_wd)), int(bool(kahan_sum)), int(update))  # fmt: skip


def radam_tail(t, update, *, lr, beta1, beta2, weight_decay, eps, decouple_wd=False, decouple_lr=False, max_lr=None,
               kahan_sum=False):  # fmt: skip
    beta2_hat = debias_beta(beta2, t)
    rect = rectification(beta2, t)
    wd = fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    return (lr, 1 - debias_beta(beta1, t), beta2_hat, 1 - beta2_hat, wd, eps, int(rect is not None),
            rect if rect is not None else 0.0, int(decouple_wd or decouple_lr), int(bool(kahan_sum)), int(update))  # fmt: skip


def ranger_tail(t, update, *, lr, beta1, beta2, weight_decay, eps, k, alpha, decouple_wd=True, decouple_lr=False, max_lr=None,
                kahan_sum=False):  # fmt: skip
    beta2_hat = debias_beta(beta2, t)
    rect = rectification(beta2, t)
    wd = fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    return (lr, 1 - debias_beta(beta1, t), beta2_hat, 1 - beta2_hat, wd, eps, int(rect is not None),
            rect if rect is not None else 0.0, int(t % k == 0), alpha, int(decouple_wd or decouple_lr), int(bool(kahan_sum)),
            int(update))  # fmt: skip
