"""Host side of one step call: tensor-list checks, grouping, pointer tables, the C-ABI call."""

from __future__ import annotations

import ctypes
from typing import Callable, Sequence

import torch
from torch import Tensor

from . import _lib

TensorList = Sequence[Tensor | None] | Tensor | None

# every call of a kernel entry point adds to this (tests and the benchmark read it)
launch_count = 0


def as_list(x: TensorList, n: int | None = None) -> list[Tensor | None] | None:
    """A bare tensor (the gradient-release form of the functional API) becomes a one-element list."""
    if x is None:
        return None
    if isinstance(x, Tensor):
        return [x]
    return list(x)


def is_dense(t: Tensor) -> bool:
    """True when the tensor's elements fill one gap-free, non-overlapping block of memory in SOME order
    of the dimensions (contiguous, channels_last, any transposition of a contiguous tensor)."""
    if t.is_contiguous():
        return True
    expected = 1
    for size, stride in sorted(((sz, st) for sz, st in zip(t.shape, t.stride()) if sz != 1), key=lambda x: x[1]):
        if stride != expected:
            return False
        expected *= size
    return True


def _dense_like(t: Tensor, ref: Tensor) -> bool:
    if t.is_contiguous() and ref.is_contiguous():
        return True
    # any dense, non-overlapping layout works as long as every tensor of the element shares it
    return t.stride() == ref.stride() and is_dense(t)


def _check_group(name: str, lists: list[list[Tensor] | None], list_names: Sequence[str]) -> None:
    params = lists[0]
    for lst, lname in zip(lists, list_names):
        if lst is None:
            continue
        for i, t in enumerate(lst):
            p = params[i]
            if not t.is_cuda:
                raise RuntimeError(
                    f"{name}: `{lname}`[{i}] lives on {t.device}; optimi_b200 steps CUDA tensors only (there is no CPU path)"
                )
            if t.device != p.device or t.dtype != p.dtype or t.numel() != p.numel():
                raise RuntimeError(
                    f"{name}: `{lname}`[{i}] ({t.dtype}, {t.device}, {t.numel()} elements) does not match its parameter "
                    f"({p.dtype}, {p.device}, {p.numel()} elements)"
                )
            if not _dense_like(t, p):
                raise RuntimeError(f"{name}: `{lname}`[{i}] must be contiguous (or share its parameter's dense layout)")


def group_by_device_and_dtype(lists: list[list[Tensor | None] | None]):
    """Splits parallel tensor lists by (device, dtype) of the first list, keeping order.

    A list whose entries are None for a group (e.g. `kahan_comps` of float32 parameters) is
    dropped to None for that group.
    """
    params = lists[0]
    keys: dict[tuple, list[int]] = {}
    for i, p in enumerate(params):
        keys.setdefault((p.device, p.dtype), []).append(i)
    if len(keys) == 1:  # the usual case: one device, one dtype — no re-slicing
        yield next(iter(keys)), [None if (lst is None or any(t is None for t in lst)) else lst for lst in lists]
        return
    for key, idx in keys.items():
        sub = []
        for lst in lists:
            if lst is None:
                sub.append(None)
                continue
            picked = [lst[i] for i in idx]
            sub.append(None if any(t is None for t in picked) else picked)
        yield key, sub


def _check_grads_only(name: str, params: list[Tensor], grads: list[Tensor]) -> None:
    """The per-step check of a trusted call: gradients are the one list the optimizer did not create."""
    for i, (p, g) in enumerate(zip(params, grads)):
        if g.dtype != p.dtype or g.device != p.device or not _dense_like(g, p):
            _check_group(name, [params, grads], ("params", "grads"))
            raise RuntimeError(f"{name}: `grads`[{i}] does not match its parameter's dtype, device or layout")


def launch(
    fn_name: str,
    lists: list[TensorList],
    list_names: Sequence[str],
    tail: Callable[[torch.device, torch.dtype, list[list[Tensor] | None]], tuple],
    stream: torch.cuda.Stream | None = None,
    trusted: bool = False,
) -> None:
    """Calls entry point `fn_name` once per (device, dtype) group of `lists`.

    `tail(device, dtype, group_lists)` returns the arguments that follow `dtype` in the C
    signature, without the trailing stream.  `trusted` (set by the optimizer classes, whose states
    are created to match their parameters and whose parameters were checked when first seen) limits
    the per-step checks to the gradients.
    """
    global launch_count
    lists = [as_list(x) for x in lists]
    if lists[0] is None or len(lists[0]) == 0:
        return
    if lists[0][0] is None:
        raise RuntimeError(f"{fn_name}: params must be tensors")
    fn = getattr(_lib.LIB, fn_name)
    for (device, dtype), sub in group_by_device_and_dtype(lists):
        if device.type != "cuda":
            raise RuntimeError(f"{fn_name}: parameters live on {device}; optimi_b200 steps CUDA tensors only (there is no CPU path)")
        if dtype not in _lib.DTYPE_CODE:
            raise RuntimeError(f"{fn_name}: unsupported parameter dtype {dtype} (float32, bfloat16 and float16 are)")
        if trusted:
            _check_grads_only(fn_name, sub[0], sub[1])
        else:
            _check_group(fn_name, sub, list_names)
        arrays = [_lib.pointer_list(x) for x in sub]
        numels = _lib.numel_array(sub[0])
        with torch.cuda.device(device):
            s = stream if stream is not None else torch.cuda.current_stream(device)
            rc = fn(
                len(sub[0]),
                *[a.ptr if a is not None else None for a in arrays],
                ctypes.cast(numels, ctypes.c_void_p),
                _lib.DTYPE_CODE[dtype],
                *tail(device, dtype, sub),
                ctypes.c_void_p(s.cuda_stream),
            )
        _lib.check(rc)
        launch_count += 1
