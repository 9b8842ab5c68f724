"""Model-side helpers kept for drop-in compatibility: weight-decay parameter groups and casting a
model to low precision with float32 islands (optimi/utils.py:41-169).  Neither touches the step
kernels; they only decide which tensors, in which dtype, the optimizers will see.
"""

from __future__ import annotations

import inspect
from collections.abc import Iterable
from typing import Any

import torch
from torch import nn

from .functional import debias, debias_beta  # noqa: F401  (re-exported like the reference's utils)


def param_groups_weight_decay(
    model: nn.Module, weight_decay: float = 1e-2, additional_layers: Iterable[str] | None = None
) -> list[dict[str, Any]]:
    """Two parameter groups: biases, 1-D tensors (norm weights) and anything whose name contains
    one of `additional_layers` get `weight_decay=0`; everything else gets `weight_decay`.
    Frozen parameters are left out.  The no-decay group comes first.
    """
    skip_names = set(additional_layers) if additional_layers is not None else set()
    groups = {False: [], True: []}
    for name, param in model.named_parameters():
        if not param.requires_grad:
            continue
        exempt = param.ndim <= 1 or name.endswith(".bias") or any(s in name for s in skip_names)
        groups[not exempt].append(param)
    return [{"params": groups[False], "weight_decay": 0.0}, {"params": groups[True], "weight_decay": weight_decay}]


def _split_buffer_spec(spec) -> tuple[set[str], tuple[type[nn.Module], ...]]:
    if spec is None:
        return set(), ()
    if not isinstance(spec, Iterable) or isinstance(spec, str):
        spec = (spec,)
    words, kinds = set(), set()
    for item in spec:
        if isinstance(item, str):
            words.add(item.lower())
        elif isinstance(item, type) and issubclass(item, nn.Module):
            kinds.add(item)
        else:
            raise TypeError("fp32_buffers items must be str or a nn.Module subclass type")
    return words, tuple(kinds)


def _module_types(spec) -> tuple[type[nn.Module], ...]:
    if spec is None:
        return ()
    if not isinstance(spec, Iterable):
        spec = (spec,)
    spec = tuple(spec)
    if not all(isinstance(t, type) and issubclass(t, nn.Module) for t in spec):
        raise TypeError("fp32_modules must be nn.Module subclass type(s)")
    return spec


def to_low_precision(
    model: nn.Module,
    dtype: torch.dtype = torch.bfloat16,
    device: torch.device | str | None = None,
    fp32_modules: type[nn.Module] | Iterable[type[nn.Module]] | None = nn.Embedding,
    fp32_buffers: str | type[nn.Module] | Iterable[str] | Iterable[type[nn.Module]] | None = ("rope", "rotary"),
) -> nn.Module:
    """Casts `model` in place to `dtype`, keeping float32 islands.

    Modules of a type in `fp32_modules` (default `nn.Embedding`) keep parameters and buffers in
    float32.  Modules whose qualified name contains a keyword of `fp32_buffers`, or whose type is
    listed there, keep only their buffers in float32 (RoPE tables).  Everything else floating
    point becomes `dtype`; `device`, if given, is applied to everything that is cast.
    """
    words, buffer_kinds = _split_buffer_spec(fp32_buffers)
    param_kinds = _module_types(fp32_modules)
    if "recurse" not in inspect.signature(nn.Module._apply).parameters:
        raise ValueError("`to_low_precision` requires PyTorch version 2.1 or newer.")

    for qualname, module in model.named_modules():
        params_stay = isinstance(module, param_kinds)
        buffers_stay = params_stay or isinstance(module, buffer_kinds) or any(w in qualname for w in words)
        own_params = {id(p) for p in module.parameters(recurse=False)}
        own_buffers = {id(b) for b in module.buffers(recurse=False)}

        def cast(t: torch.Tensor, ids, stay):
            if id(t) in ids and t.is_floating_point():
                return t.to(dtype=torch.float32 if stay else dtype, device=device)
            return t

        # Module._apply swaps parameters/buffers (and their grads) the way .to() does
        module._apply(lambda t: cast(t, own_params, params_stay), recurse=False)
        module._apply(lambda t: cast(t, own_buffers, buffers_stay), recurse=False)
    return model
