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

import ctypes

import torch
from torch import Tensor

from . import _lib
from . import _tails as T
from ._launch import TensorList, launch
from ._tails import debias, debias_beta  # noqa: F401  (part of the reference's utils API)

__all__ = ["adam", "adamw", "lion", "sgd", "stableadamw", "adan", "radam", "ranger", "debias", "debias_beta"]


def _advance(step: Tensor) -> int:
    step.add_(1)
    return int(step.item())


def _check_release(gradient_release: bool, foreach: bool, triton: bool) -> None:
    """The one combination of back-end keywords the reference rejects (e.g. optimi/adam.py:278-282): the
    per-parameter form of a step asked for together with the foreach back end and without Triton."""
    if gradient_release and foreach and not triton:
        raise ValueError(f"Gradient release {gradient_release=} and foreach {foreach=} cannot be used together")


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
):
    """Adam / AdamW step on lists of tensors (or bare tensors in gradient-release form)."""
    t = _advance(step)
    _check_release(gradient_release, foreach, triton)
    tail = T.adam_tail(t, not optimizer_accumulation, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, eps=eps,
                       decouple_wd=decouple_wd, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum)  # fmt: skip
    lists = [params, grads, exp_avgs, exp_avg_sqs, kahan_comps]
    names = ("params", "grads", "exp_avgs", "exp_avg_sqs", "kahan_comps")
    launch("optimi_b200_adam", lists, names, lambda *_: tail, _stream, _trusted)


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
):
    """AdamW step: `adam` with decoupled weight decay (optimi/adamw.py:123-143)."""
    adam(
        params, grads, exp_avgs, exp_avg_sqs, kahan_comps, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay,
        eps=eps, step=step, decouple_wd=True, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum,
        foreach=foreach, triton=triton, gradient_release=gradient_release, optimizer_accumulation=optimizer_accumulation, _stream=_stream, _trusted=_trusted,
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
    _check_release(gradient_release, foreach, triton)
    tail = T.lion_tail(0, not optimizer_accumulation, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay,
                       decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum)  # fmt: skip
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
    _check_release(gradient_release, foreach, triton)
    if momentum == 0:
        exp_avgs = None
    tail = T.sgd_tail(0, not optimizer_accumulation, lr=lr, momentum=momentum, weight_decay=weight_decay, dampening=dampening,
                      decouple_wd=decouple_wd, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum)  # fmt: skip
    launch("optimi_b200_sgd", [params, grads, exp_avgs, kahan_comps], ("params", "grads", "exp_avgs", "kahan_comps"),
           lambda *_: tail, _stream, _trusted)  # fmt: skip


_workspaces: dict[tuple, Tensor] = {}
_outgrown: list[Tensor] = []


def _stable_workspace(device: torch.device, stream_id: int, nbytes: int) -> Tensor:
    """Device scratch for StableAdamW's per-chunk partial sums (and the gradient-norm passes), cached per
    (device, stream) and grown on demand, so steady-state steps allocate nothing.  A buffer that has been
    outgrown is kept for the life of the process instead of being handed back to the allocator: kernels
    already enqueued on a side stream, or launches captured into a CUDA graph, may still name it, and the
    allocator knows nothing about either (the buffers are used on raw stream handles).  They are small
    (8 bytes per 512 elements of the largest list) and grow a handful of times at most."""
    key = (device, stream_id)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _outgrown.append(ws)
        ws = torch.empty(max(2 * nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def stable_workspace_args(device: torch.device, stream_ptr: int, params) -> tuple:
    """(pointer, size) of the cached scratch StableAdamW's reduction needs for this tensor list."""
    numels = _lib.numel_array(params)
    need = _lib.LIB.optimi_b200_stableadamw_workspace_bytes(len(params), ctypes.cast(numels, ctypes.c_void_p))
    ws = _stable_workspace(device, stream_ptr, need)
    return (ctypes.c_void_p(ws.data_ptr()), ws.numel())


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
    t = _advance(step)
    _check_release(gradient_release, foreach, triton)
    update = not optimizer_accumulation
    scalars = T.stableadamw_tail(t, update, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, eps=eps,
                                 decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum)  # fmt: skip

    def tail(device, dtype, sub):
        if not update:
            return scalars + (None, 0)
        s = _stream if _stream is not None else torch.cuda.current_stream(device)
        return scalars + stable_workspace_args(device, s.cuda_stream, sub[0])

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
    _check_release(gradient_release, foreach, triton)
    tail = T.adan_tail(t, not optimizer_accumulation, lr=lr, beta1=beta1, beta2=beta2, beta3=beta3, weight_decay=weight_decay,
                       eps=eps, decouple_lr=decouple_lr, max_lr=max_lr, adam_wd=adam_wd, kahan_sum=kahan_sum)  # fmt: skip
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
    _check_release(gradient_release, foreach, triton)
    tail = T.radam_tail(t, not optimizer_accumulation, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, eps=eps,
                        decouple_wd=decouple_wd, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum)  # fmt: skip
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
    _check_release(gradient_release, foreach, triton)
    tail = T.ranger_tail(t, not optimizer_accumulation, lr=lr, beta1=beta1, beta2=beta2, weight_decay=weight_decay, eps=eps,
                         k=k, alpha=alpha, decouple_wd=decouple_wd, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum)  # fmt: skip
    launch(
        "optimi_b200_ranger", [params, grads, exp_avgs, exp_avg_sqs, la_params, kahan_comps],
        ("params", "grads", "exp_avgs", "exp_avg_sqs", "la_params", "kahan_comps"), lambda *_: tail, _stream, _trusted,
    )  # fmt: skip
