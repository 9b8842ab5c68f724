"""Gradient release: step each parameter inside the backward pass, then drop its gradient.

Same user-facing functions and checks as the reference (optimi/gradientrelease.py:13-61).  The
hook itself is the reference's — `optimizer.step(param=p)` followed by `optimizer.zero_grad(param=p)`
— and what differs is underneath: the per-parameter step is one small launch of the same
multi-tensor kernel, by default on a side stream so that it overlaps the rest of the backward pass
(`side_stream=` here, `OptimiOptimizer.use_release_stream` to change it later).
"""

from __future__ import annotations

from warnings import warn

from torch import Tensor
from torch.nn import Module

from .optimizer import OptimiOptimizer

_HOOKS_ATTR = "_gradient_release_hooks"


class _ReleaseHook:
    """Callable registered as a post-accumulate-grad hook."""

    __slots__ = ("optimizer",)

    def __init__(self, optimizer: OptimiOptimizer):
        self.optimizer = optimizer

    def __call__(self, param: Tensor) -> None:
        # what the reference's hook does — optimizer.step(param=param); optimizer.zero_grad(param=param)
        # (optimi/gradientrelease.py:13-15) — without the two method-call wrappers
        self.optimizer._release(param)
        param.grad = None


def prepare_for_gradient_release(model: Module, optimizer: OptimiOptimizer, ignore_existing_hooks: bool = False,
                                 side_stream: bool = True):  # fmt: skip
    """Registers a post-accumulate-grad hook on every trainable parameter of `model` that steps it
    with `optimizer` (which must have been created with `gradient_release=True`) and frees its
    gradient.  Refuses to stack on top of other post-accumulate-grad hooks unless
    `ignore_existing_hooks=True`.

    `side_stream=True` (the default, for CUDA models) runs the released steps on a stream of their own:
    each step waits for the gradient it consumes, and the stream that runs the backward pass waits for
    all released steps when the backward pass ends, so code after `loss.backward()` sees updated
    parameters as before.  A stream chosen earlier with `optimizer.use_release_stream(...)` is kept;
    `side_stream=False` steps on the stream the hook fires on, as the reference does.
    """
    if not isinstance(optimizer, OptimiOptimizer):
        raise TypeError("`optimizer` must be an instance of `OptimiOptimizer`")
    if not optimizer.defaults["gradient_release"]:
        raise ValueError("`optimizer` must be initialized with `gradient_release=True`")

    trainable = [p for p in model.parameters() if p.requires_grad]
    if not ignore_existing_hooks:
        for p in trainable:
            if p._post_accumulate_grad_hooks is not None and len(p._post_accumulate_grad_hooks) > 0:
                raise ValueError(
                    "Model already has post_accumulate_grad_hooks. If this is expected, rerun with `ignore_existing_hooks=True`."
                )
    if side_stream and optimizer._release_stream is None and not optimizer._release_stream_chosen and any(p.is_cuda for p in trainable):
        optimizer.use_release_stream(True)
    hook = _ReleaseHook(optimizer)
    setattr(model, _HOOKS_ATTR, [p.register_post_accumulate_grad_hook(hook) for p in trainable])


def remove_gradient_release(model: Module):
    """Removes the hooks `prepare_for_gradient_release` registered on `model`."""
    handles = getattr(model, _HOOKS_ATTR, None)
    if handles is None:
        warn("`model` does not have any gradient release post_accumulate_grad_hooks to remove.")
        return
    for h in handles:
        if hasattr(h, "remove"):
            h.remove()
    delattr(model, _HOOKS_ATTR)
