"""Functional step API: adam, adamw, lion, sgd, stableadamw, adan, radam, ranger.

Same signatures and host-side scalar arithmetic as the reference's functional entry points
(optimi/adam.py:213-309, adamw.py:78-143, lion.py:187-266, sgd.py:214-292, stableadamw.py:277-371,
adan.py:236-350, radam.py:214-321, ranger.py:229-346); where the reference then picks a
`_single_*`, `_foreach_*` or `_triton_*` back end, these call one sm_100a multi-tensor kernel
through the C ABI.  The `foreach` and `triton` keywords are accepted and ignored (one back end),
`gradient_release` only changes the accepted argument form (bare tensors instead of lists).

Scalars are computed as Python doubles in the reference's order of operations so that the fp32
values the kernels receive are the ones the reference's ATen ops receive.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor

from . import _lib
from ._launch import TensorList, as_list, launch

__all__ = ["adam", "adamw", "lion", "sgd", "stableadamw", "adan", "radam", "ranger", "debias", "debias_beta"]


def debias(beta: float, step: int) -> float:
    """Adam's bias-correction denominator 1 - beta^step (optimi/utils.py:26-28)."""
    return 1 - beta**step


def debias_beta(beta: float, step: int) -> float:
    """Beta with the bias correction folded in, beta*(1-beta^(step-1))/(1-beta^step) in the
    reference's simplified form (optimi/utils.py:31-36); 0 at step 1."""
    return (beta**step - beta) / (beta**step - 1)


def _advance(step: Tensor) -> int:
    step.add_(1)
    return int(step.item())


def _fold_weight_decay(weight_decay: float, lr: float, decouple_wd: bool, decouple_lr: bool, max_lr: float | None) -> float:
    """The multiplicative factor for (fully) decoupled decay, or the raw L2 coefficient."""
    if weight_decay != 0:
        if decouple_lr:
            return 1 - (lr / max_lr) * weight_decay
        if decouple_wd:
            return 1 - lr * weight_decay
    return weight_decay


def _rectification(beta2: float, step: int) -> float | None:
    """RAdam's variance rectification term; None while the SMA length is at most 5."""
    rho_inf = 2 / (1 - beta2) - 1
    rho = rho_inf - 2 * step * (beta2**step) / debias(beta2, step)
    if rho > 5:
        return math.sqrt(((rho - 4) * (rho - 2) * rho_inf) / ((rho_inf - 4) * (rho_inf - 2) * rho))
    return None


def _kahan(kahan_sum: bool, kahan_comps) -> bool:
    return bool(kahan_sum) and kahan_comps is not None


def adam(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    exp_avg_sqs: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    weight_decay: float,
    eps: float,
    step: Tensor,
    decouple_wd: bool,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
    _push=None,
):
    """Adam / AdamW step on lists of tensors (or bare tensors in gradient-release form).

    `_push` (a sequence of byte offsets to the peers' copies of the parameter buffer) selects the
    fused step + exchange kernel of a sharded run; see `optimi_b200.zero.ShardedOptimizer`.
    """
    t = _advance(step)
    beta1_comp = 1 - debias_beta(beta1, t)
    beta2_hat = debias_beta(beta2, t)
    beta2_comp = 1 - beta2_hat
    wd = _fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    if _push is not None and not optimizer_accumulation:
        import ctypes

        deltas = (ctypes.c_int64 * len(_push))(*_push)
        tail = (lr, beta1_comp, beta2_hat, beta2_comp, wd, eps, int(decouple_wd or decouple_lr), int(bool(kahan_sum)),
                len(_push), ctypes.cast(deltas, ctypes.c_void_p))  # fmt: skip
        launch(
            "optimi_b200_adam_push", [params, grads, exp_avgs, exp_avg_sqs, kahan_comps],
            ("params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"), lambda *_: tail, _stream, _trusted,
        )  # fmt: skip
        return
    tail = (lr, beta1_comp, beta2_hat, beta2_comp, wd, eps, int(decouple_wd or decouple_lr), int(bool(kahan_sum)),
            int(not optimizer_accumulation))  # fmt: skip
    launch(
        "optimi_b200_adam", [params, grads, exp_avgs, exp_avg_sqs, kahan_comps],
        ("params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"), lambda *_: tail, _stream, _trusted,
    )  # fmt: skip


def adamw(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    exp_avg_sqs: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    weight_decay: float,
    eps: float,
    step: Tensor,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
    _push=None,
):
    """AdamW step: `adam` with decoupled weight decay (optimi/adamw.py:123-143)."""
    adam(
        params, grads, exp_avgs, exp_avg_sqs, kahan_comps, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay,
        eps=eps, step=step, decouple_wd=True, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum,
        gradient_release=gradient_release, optimizer_accumulation=optimizer_accumulation, _stream=_stream, _trusted=_trusted, _push=_push,
    )  # fmt: skip


def lion(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    weight_decay: float,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
):
    """Lion step.  Weight decay is always decoupled (optimi/lion.py:227-231)."""
    wd = _fold_weight_decay(weight_decay, lr, True, decouple_lr, max_lr)
    tail = (lr, 1 - beta1, 1 - beta2, wd, int(bool(kahan_sum)), int(not optimizer_accumulation))
    launch("optimi_b200_lion", [params, grads, exp_avgs, kahan_comps], ("params", "grads", "exp_avgs", "kahan_comps"),
           lambda *_: tail, _stream, _trusted)  # fmt: skip


def sgd(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    momentum: float,
    weight_decay: float,
    dampening: bool,
    decouple_wd: bool,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
):
    """SGD step with optional momentum, dampening and (decoupled) weight decay."""
    wd = _fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    if momentum == 0:
        exp_avgs = None
    tail = (lr, momentum, wd, int(bool(dampening)), int(decouple_wd or decouple_lr), int(bool(kahan_sum)),
            int(not optimizer_accumulation))  # fmt: skip
    launch("optimi_b200_sgd", [params, grads, exp_avgs, kahan_comps], ("params", "grads", "exp_avgs", "kahan_comps"),
           lambda *_: tail, _stream, _trusted)  # fmt: skip


_workspaces: dict[tuple, Tensor] = {}


def _stable_workspace(device: torch.device, stream_id: int, nbytes: int) -> Tensor:
    """Device scratch for StableAdamW's per-chunk partial sums, cached per (device, stream) and grown
    on demand, so steady-state steps allocate nothing."""
    key = (device, stream_id)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def stableadamw(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    exp_avg_sqs: TensorList,
    eps_sqs: TensorList = None,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    weight_decay: float,
    eps: float,
    step: Tensor,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    mean_squares: TensorList = None,
    _stream=None,
    _trusted: bool = False,
):
    """StableAdamW step.  `eps_sqs` and `mean_squares` are accepted for signature compatibility; the
    kernels derive eps^2 from `eps` and keep the per-tensor mean square in their own scratch."""
    import ctypes

    t = _advance(step)
    beta1_comp = 1 - debias_beta(beta1, t)
    beta2_hat = debias_beta(beta2, t)
    beta2_comp = 1 - beta2_hat
    update = not optimizer_accumulation

    def tail(device, dtype, sub):
        ws_ptr, ws_bytes = None, 0
        if update:
            numels = _lib.numel_array(sub[0])
            need = _lib.LIB.optimi_b200_stableadamw_workspace_bytes(len(sub[0]), ctypes.cast(numels, ctypes.c_void_p))
            s = _stream if _stream is not None else torch.cuda.current_stream(device)
            ws = _stable_workspace(device, s.cuda_stream, need)
            ws_ptr, ws_bytes = ctypes.c_void_p(ws.data_ptr()), ws.numel()
        return (lr, beta1_comp, beta2_hat, beta2_comp, weight_decay, eps, int(bool(decouple_lr)),
                float(max_lr) if max_lr is not None else 0.0, int(bool(kahan_sum)), int(update), ws_ptr, ws_bytes)  # fmt: skip

    launch(
        "optimi_b200_stableadamw", [params, grads, exp_avgs, exp_avg_sqs, kahan_comps],
        ("params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"), tail, _stream, _trusted,
    )  # fmt: skip


def adan(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    exp_avg_diffs: TensorList,
    exp_avg_sqs: TensorList,
    prev_grads: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    beta3: float,
    weight_decay: float,
    eps: float,
    step: Tensor,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    adam_wd: bool = False,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
):
    """Adan step.  `prev_grads` holds the negated previous gradient."""
    t = _advance(step)
    beta1_comp = 1 - debias_beta(beta1, t)
    beta2_comp = 1 - debias_beta(beta2, t)
    beta3_hat = debias_beta(beta3, t)
    beta3_comp = 1 - beta3_hat
    wd = weight_decay
    if wd != 0:
        wd = (lr / max_lr) * wd if decouple_lr else lr * wd
        wd = 1 - wd if adam_wd else 1 + wd
    tail = (lr, beta1_comp, beta2, beta2_comp, beta3_hat, beta3_comp, eps, wd, int(bool(adam_wd)), int(bool(kahan_sum)),
            int(not optimizer_accumulation))  # fmt: skip
    launch(
        "optimi_b200_adan", [params, grads, exp_avgs, exp_avg_diffs, exp_avg_sqs, prev_grads, kahan_comps],
        ("params", "grads", "exp_avgs", "exp_avg_diffs", "exp_avg_sqs", "prev_grads", "kahan_comps"), lambda *_: tail, _stream, _trusted,
    )  # fmt: skip


def radam(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    exp_avg_sqs: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    weight_decay: float,
    eps: float,
    step: Tensor,
    decouple_wd: bool = False,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
):
    """RAdam step: Adam averages with a rectified step once the variance estimate is trusted."""
    t = _advance(step)
    beta1_comp = 1 - debias_beta(beta1, t)
    beta2_hat = debias_beta(beta2, t)
    beta2_comp = 1 - beta2_hat
    rect = _rectification(beta2, t)
    wd = _fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    tail = (lr, beta1_comp, beta2_hat, beta2_comp, wd, eps, int(rect is not None), rect if rect is not None else 0.0,
            int(decouple_wd or decouple_lr), int(bool(kahan_sum)), int(not optimizer_accumulation))  # fmt: skip
    launch(
        "optimi_b200_radam", [params, grads, exp_avgs, exp_avg_sqs, kahan_comps],
        ("params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps"), lambda *_: tail, _stream, _trusted,
    )  # fmt: skip


def ranger(
    params: TensorList,
    grads: TensorList,
    exp_avgs: TensorList,
    exp_avg_sqs: TensorList,
    la_params: TensorList,
    kahan_comps: TensorList = None,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    weight_decay: float,
    eps: float,
    k: int,
    alpha: float,
    step: Tensor,
    decouple_wd: bool = True,
    decouple_lr: bool = False,
    max_lr: float | None = None,
    kahan_sum: bool = False,
    foreach: bool = False,
    triton: bool = False,
    gradient_release: bool = False,
    optimizer_accumulation: bool = False,
    _stream=None,
    _trusted: bool = False,
):
    """Ranger step: RAdam followed, on every k-th step, by a Lookahead pull toward the slow weights."""
    t = _advance(step)
    beta1_comp = 1 - debias_beta(beta1, t)
    beta2_hat = debias_beta(beta2, t)
    beta2_comp = 1 - beta2_hat
    rect = _rectification(beta2, t)
    wd = _fold_weight_decay(weight_decay, lr, decouple_wd, decouple_lr, max_lr)
    tail = (lr, beta1_comp, beta2_hat, beta2_comp, wd, eps, int(rect is not None), rect if rect is not None else 0.0,
            int(t % k == 0), alpha, int(decouple_wd or decouple_lr), int(bool(kahan_sum)), int(not optimizer_accumulation))  # fmt: skip
    launch(
        "optimi_b200_ranger", [params, grads, exp_avgs, exp_avg_sqs, la_params, kahan_comps],
        ("params", "grads", "exp_avgs", "exp_avg_sqs", "la_params", "kahan_comps"), lambda *_: tail, _stream, _trusted,
    )  # fmt: skip
