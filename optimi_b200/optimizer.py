"""Optimizer classes with the reference's constructor, `step`, `zero_grad`, `state_dict` and
gradient-release / optimizer-accumulation behaviour, stepping through the sm_100a kernels.

One base class does all bookkeeping from a small per-optimizer description (which state tensors
exist and how they start, which hyper-parameters go to the functional call); the reference spells
the same logic out once per optimizer (optimi/optimizer.py:12-114 plus `_init_state`, `_init_group`
and `step` of each optimi/<optimizer>.py).  What a checkpoint sees is unchanged: state keys, dtypes
and shapes, `param_groups` entries including `setup` and the int32 CPU `step` tensor.
"""

from __future__ import annotations

from collections.abc import Callable, Iterable
from typing import Any
from warnings import warn

import torch
from torch import Tensor
from torch.optim.optimizer import Optimizer

import ctypes

from . import _lib
from . import _tails as T
from . import functional as F
from ._launch import _dense_like, is_dense

LOW_PRECISION = (torch.float16, torch.bfloat16)


def _check_range(name: str, value: float, shown: str | None = None):
    if not 0.0 <= value < 1.0:
        raise ValueError(f"Invalid {name} parameter: {shown or name}={value}")


def _check_gradient(fn_name: str, grad: Tensor, param: Tensor) -> None:
    """The kernels pair the elements of a gradient and its parameter by position in memory, so the two
    must agree in dtype, device and memory layout (both contiguous, or the same dense strides: a
    channels_last parameter needs a channels_last gradient)."""
    if grad.dtype != param.dtype or grad.device != param.device or not _dense_like(grad, param):
        raise RuntimeError(f"{fn_name}: a gradient does not match its parameter's dtype, device or layout")


class _ReleasePlan:
    """Prebuilt C arguments for stepping one parameter (gradient release).  Valid while the parameter
    and its state tensors stay where they are; only the gradient pointer changes from call to call."""

    __slots__ = ("fn_name", "fn", "group", "device", "index", "dtype_code", "tensors", "addresses", "arrays", "args",
                 "grad_slot", "numels", "numels_arg", "step_view")  # fmt: skip

    def __init__(self, fn_name: str, param: Tensor, group: dict, states: list, step: Tensor | None):
        self.fn_name, self.fn, self.group = fn_name, getattr(_lib.LIB, fn_name), group
        self.device, self.index = param.device, param.device.index
        self.dtype_code = _lib.DTYPE_CODE[param.dtype]
        self.tensors = [param] + states
        for t in states:
            if t is not None and (t.device != param.device or t.dtype != param.dtype or t.numel() != param.numel() or not _dense_like(t, param)):
                raise RuntimeError(f"{fn_name}: a state tensor does not match its parameter's dtype, device, size or layout")
        self.addresses = [None if t is None else t.data_ptr() for t in self.tensors]
        # C order: params, grads, states...
        self.grad_slot = (ctypes.c_void_p * 1)(0)
        self.arrays = [(ctypes.c_void_p * 1)(self.addresses[0]), self.grad_slot] + [
            None if a is None else (ctypes.c_void_p * 1)(a) for a in self.addresses[1:]
        ]
        self.args = [None if a is None else ctypes.cast(a, ctypes.c_void_p) for a in self.arrays]
        self.numels = (ctypes.c_int64 * 1)(param.numel())
        self.numels_arg = ctypes.cast(self.numels, ctypes.c_void_p)
        # the int32 CPU counter of the checkpoint layout, advanced in place through a numpy view
        self.step_view = None if step is None else step.numpy()

    def fresh(self, param: Tensor) -> bool:
        for t, a in zip(self.tensors, self.addresses):
            if (None if t is None else t.data_ptr()) != a:
                return False
        return True


class _SubPlan:
    """The tensors of one (device, dtype) of a parameter group with their C pointer tables."""

    __slots__ = ("fn_name", "fn", "n", "device", "index", "dtype_code", "params", "fixed", "addresses", "arrays", "args",
                 "grad_array", "numels", "numels_arg")  # fmt: skip

    def __init__(self, fn_name: str, params: list[Tensor], state_lists: list[list | None]):
        p0 = params[0]
        if not p0.is_cuda:
            raise RuntimeError(f"{fn_name}: parameters live on {p0.device}; optimi_b200 steps CUDA tensors only (there is no CPU path)")
        if p0.dtype not in _lib.DTYPE_CODE:
            raise RuntimeError(f"{fn_name}: unsupported parameter dtype {p0.dtype} (float32, bfloat16 and float16 are)")
        self.fn_name, self.fn, self.n = fn_name, getattr(_lib.LIB, fn_name), len(params)
        self.device, self.index, self.dtype_code = p0.device, p0.device.index, _lib.DTYPE_CODE[p0.dtype]
        self.params = params
        for lst in state_lists:
            if lst is None:
                continue
            for t, p in zip(lst, params):
                if t.device != p.device or t.dtype != p.dtype or t.numel() != p.numel() or not _dense_like(t, p):
                    raise RuntimeError(f"{fn_name}: a state tensor does not match its parameter's dtype, device, size or layout")
        self.fixed = [t for lst in [params] + state_lists if lst is not None for t in lst]  # everything but gradients
        self.addresses = list(map(Tensor.data_ptr, self.fixed))
        self.grad_array = (ctypes.c_void_p * self.n)()
        self.arrays = [_lib.PointerArray(params).arr, self.grad_array] + [None if lst is None else _lib.PointerArray(lst).arr for lst in state_lists]
        self.args = [None if a is None else ctypes.cast(a, ctypes.c_void_p) for a in self.arrays]
        self.numels = _lib.numel_array(params)
        self.numels_arg = ctypes.cast(self.numels, ctypes.c_void_p)

    def fresh(self) -> bool:
        return list(map(Tensor.data_ptr, self.fixed)) == self.addresses

    def launch(self, tail: tuple, needs_workspace: bool) -> None:
        grads = [p.grad for p in self.params]
        for g, p in zip(grads, self.params):
            _check_gradient(self.fn_name, g, p)
        self.grad_array[:] = list(map(Tensor.data_ptr, grads))
        stream_ptr = torch._C._cuda_getCurrentRawStream(self.index)
        if needs_workspace:
            tail = tail + F.stable_workspace_args(self.device, stream_ptr, self.params)
        if torch._C._cuda_getDevice() == self.index:
            rc = self.fn(self.n, *self.args, self.numels_arg, self.dtype_code, *tail, stream_ptr)
        else:
            with torch.cuda.device(self.device):
                rc = self.fn(self.n, *self.args, self.numels_arg, self.dtype_code, *tail, stream_ptr)
        if rc != 0:
            _lib.check(rc)


class _GroupPlan:
    """Cached pointer tables for the whole-list step of one parameter group (one _SubPlan per device and dtype)."""

    __slots__ = ("key", "subs")

    def __init__(self, opt: "OptimiOptimizer", group: dict, params: list[Tensor], key: tuple):
        self.key = key
        buckets: dict[tuple, list[Tensor]] = {}
        for p in params:
            buckets.setdefault((p.device, p.dtype), []).append(p)
        self.subs = []
        for plist in buckets.values():
            state_lists = []
            for k in opt._c_states:
                lst = [opt.state[p][k] for p in plist]
                state_lists.append(None if any(t is None for t in lst) else lst)
            self.subs.append(_SubPlan(opt._c_fn, plist, state_lists))

    def fresh(self) -> bool:
        return all(sub.fresh() for sub in self.subs)


class OptimiOptimizer(Optimizer):
    """Common behaviour of every optimi_b200 optimizer (mirror of optimi/optimizer.py:12-114)."""

    # ---- per-optimizer description, overridden by subclasses ---------------------------------
    _counts_steps = True  # keeps a `step` counter (Lion and SGD do not)
    _c_fn: str = ""  # C entry point
    _c_states: tuple[str, ...] = ()  # state keys in the order of the C signature (after params, grads)
    _tail: Callable = None  # host scalars -> C arguments (optimi_b200._tails)
    _needs_workspace = False
    _scalar_keys: tuple[str, ...] = ()  # param_group keys forwarded as keywords

    def __init__(self, params: Iterable[Tensor] | Iterable[dict], defaults: dict[str, Any]):
        if not 0.0 <= defaults["lr"]:
            raise ValueError(f"Invalid learning rate: lr={defaults['lr']}")
        if not 0.0 <= defaults["weight_decay"]:
            raise ValueError(f"Invalid weight decay: weight_decay={defaults['weight_decay']}")
        if defaults["decouple_lr"] and defaults["max_lr"] is None:
            defaults["max_lr"] = defaults["lr"]
        if defaults["max_lr"] is not None and not 0.0 <= defaults["max_lr"]:
            raise ValueError(f"Invalid maximum learning rate: max_lr={defaults['max_lr']}")

        if defaults["foreach"]:
            warn(
                "Parameter `foreach` is deprecated and has no effect: optimi_b200 always steps with its CUDA multi-tensor "
                "kernels. Set `foreach=False` to silence this warning.",
                category=DeprecationWarning,
            )

        super().__init__(params, defaults)

        if self.defaults.get("decouple_lr", False):
            high = [
                g["weight_decay"]
                for g in self.param_groups
                if g.get("decouple_lr", self.defaults.get("decouple_lr", False)) and g.get("weight_decay", 0.0) >= 1e-3
            ]
            if high:
                warn(
                    f"You are using weight_decay up to {max(high)} which is potentially high for decouple_lr=True"
                    f". Unlike decoupled weight decay, fully decoupled weight decay does not reduce weight decay by the learning rate.",
                    category=UserWarning,
                )

        self._optimizer_accumulation = False
        self._plans: dict[Tensor, _ReleasePlan] = {}  # gradient release: cached C arguments per parameter
        self._tail_cache: dict[int, tuple] = {}  # id(group) -> (key, tail): scalars are shared by a group's parameters
        self._group_plans: dict[int, _GroupPlan | None] = {}  # id(group) -> cached pointer tables of the whole-list step
        self.register_load_state_dict_post_hook(lambda opt: opt._drop_plans())
        self._release_stream: torch.cuda.Stream | None = None
        self._release_stream_chosen = False  # use_release_stream was called: prepare_for_gradient_release keeps that choice
        self._release_fence_queued = False
        self._graph_nodes: _lib.GraphNodes | None = None  # kernel nodes of the step captured into a CUDA graph
        self._grad_factor: Tensor | None = None  # device scalar the next step(s) multiply the gradients by
        self._grad_factor_once = False  # set by clip_grad_norm: the factor belongs to the next step only
        self._clip_out: Tensor | None = None  # (factor, total norm) written by clip_grad_norm

        if self.defaults["gradient_release"]:
            if self.defaults["foreach"]:
                warn("Gradient release (gradient_release=True) and foreach (foreach=True) cannot be used together. Disabling foreach.", category=UserWarning)  # fmt: skip  # noqa: E501
            self.defaults["foreach"] = False
            for group in self.param_groups:
                group["foreach"] = False
                for p in group["params"]:
                    self.state[p]["group"] = group

    def _drop_plans(self) -> None:
        """Forget every cached pointer table (state tensors were replaced)."""
        self._plans.clear()
        self._group_plans.clear()
        self._tail_cache.clear()

    # ---- optimizer accumulation ---------------------------------------------------------------
    @property
    def optimizer_accumulation(self) -> bool:
        "Accumulate gradients in optimizer states during gradient release instead of a full step."
        return self._optimizer_accumulation

    @optimizer_accumulation.setter
    def optimizer_accumulation(self, optimizer_accumulation: bool):
        self._optimizer_accumulation = optimizer_accumulation

    # ---- state -------------------------------------------------------------------------------
    def _new_state(self, group: dict[str, Any], state: dict[str, Any], param: Tensor) -> None:
        """Creates the optimizer-specific state tensors of `param` (subclass hook)."""
        raise NotImplementedError

    def _first_gradient(self, param: Tensor) -> Tensor:
        """A copy of `param.grad` as the step kernels will see it — times the gradient factor when one is set —
        for the states that start from the first gradient (Adan's previous gradient, SGD's `torch_init`)."""
        grad = param.grad.detach()
        if self._grad_factor is None:
            return grad.clone()
        return (grad.float() * self._grad_factor.to(grad.device)).to(grad.dtype)  # fp32 product, one rounding: the kernels' arithmetic

    def _state_needs_first_gradient(self, group: dict[str, Any]) -> bool:
        """Whether `_new_state` reads the parameter's first gradient (Adan, SGD with `torch_init`)."""
        return False

    def _kahan_state(self, group: dict[str, Any], param: Tensor) -> Tensor | None:
        """Kahan compensation buffer: on by default for bf16/fp16 parameters (`kahan_sum=None`),
        never for float32 (e.g. optimi/adam.py:100-106)."""
        if (group["kahan_sum"] or group["kahan_sum"] is None) and param.dtype in LOW_PRECISION:
            group["kahan_sum"] = True
            return torch.zeros_like(param, memory_format=torch.preserve_format)
        return None

    def _init_state(self, group: dict[str, Any], state: dict[str, Any], param: Tensor) -> None:
        if "kahan_comp" in state:
            return
        if not param.is_contiguous() and not is_dense(param):
            raise RuntimeError("optimi_b200 needs dense parameters (contiguous or any permutation of contiguous)")
        self._new_state(group, state, param)
        state["kahan_comp"] = self._kahan_state(group, param)
        if group["gradient_release"] and self._counts_steps:
            state["step"] = torch.tensor(0, dtype=torch.int32)

    def _setup_group(self, group: dict[str, Any]) -> None:
        if not group["setup"]:
            group["setup"] = True
            if self._counts_steps:
                group["step"] = torch.tensor(0, dtype=torch.int32)

    # ---- step --------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure: Callable | None = None, param: Tensor | None = None):
        """Performs a single optimization step on the whole model or on one parameter.

        Args:
            closure: A closure which reevaluates the model and returns the loss. Incompatible with
                stepping a single `param`.
            param: One parameter to step during the backward pass. Requires `gradient_release=True`
                and hooks registered by `prepare_for_gradient_release`. Incompatible with `closure`.
        """
        loss = None
        if closure is not None and param is None:
            with torch.enable_grad():
                loss = closure()

        if param is not None:
            self._release(param)
            return loss
        factor = self._grad_factor
        if factor is not None:
            _lib.LIB.optimi_b200_grad_scale_begin(factor.data_ptr())
        try:
            if torch.cuda.is_initialized() and torch.cuda.is_current_stream_capturing():
                self._capture_step()
            else:
                for group in self.param_groups:
                    self._step_group(group)
        finally:
            if factor is not None:
                _lib.LIB.optimi_b200_grad_scale_end()
                if self._grad_factor_once:
                    self._grad_factor = None
        return loss

    @torch.no_grad()
    def step_groups(self, indices: Iterable[int]) -> None:
        """Steps only the parameter groups `param_groups[i]` for i in `indices` (each group keeps its own
        step counter, so groups may be stepped at different moments): a caller whose gradients arrive in
        pieces — copied in from the host, or reduced bucket by bucket — can step each piece as soon as it is
        complete instead of waiting for the last one.  One call of `step()` equals `step_groups` over all
        groups.  Not for a capturing stream."""
        if torch.cuda.is_initialized() and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("step_groups cannot be captured into a CUDA graph; capture step()")
        factor = self._grad_factor
        if factor is not None:
            _lib.LIB.optimi_b200_grad_scale_begin(factor.data_ptr())
        try:
            for i in indices:
                self._step_group(self.param_groups[i])
        finally:
            if factor is not None:
                _lib.LIB.optimi_b200_grad_scale_end()

    # ---- gradient scaling fused into the step ----------------------------------------------------
    def set_grad_factor(self, factor: Tensor | None) -> None:
        """From now on every step multiplies each gradient element by `factor` (a CUDA float32 tensor with
        one element, read on the device when the step runs) as it loads it: `g <- round(g * factor)`, what
        `torch._foreach_mul_(grads, factor)` would have done in a pass of its own — a GradScaler's inverse
        scale, a clip coefficient computed elsewhere.  The gradients themselves are left as they are.
        `None` switches it off.  Also applies to gradient-release steps."""
        if factor is not None and (factor.dtype != torch.float32 or not factor.is_cuda or factor.numel() != 1):
            raise ValueError("set_grad_factor: the factor must be a CUDA float32 tensor with one element")
        self._grad_factor, self._grad_factor_once = factor, False

    @torch.no_grad()
    def clip_grad_norm(self, max_norm: float) -> Tensor:
        """`torch.nn.utils.clip_grad_norm_(params, max_norm)` without touching the gradients: computes
        the total 2-norm of all gradients and the clip coefficient `min(1, max_norm / (norm + 1e-6))`
        on the device (one read of the gradients, PyTorch's own order of roundings), and makes the
        NEXT `step()` scale the gradients by the coefficient as it loads them.  Returns the total norm
        as a 0-dim CUDA tensor (no host synchronisation).  Saves the read-modify-write pass over the
        gradients that clipping in place costs.  All gradients must live on one device; not for gradient
        release, where parameters are stepped before all gradients exist."""
        if self.defaults.get("gradient_release", False):
            raise RuntimeError("clip_grad_norm needs all gradients before any parameter is stepped: not with gradient_release")
        grads = [p.grad for group in self.param_groups for p in group["params"] if p.grad is not None]
        if not grads:
            raise RuntimeError("clip_grad_norm: no parameter has a gradient")
        g0 = grads[0]
        if not g0.is_cuda or g0.dtype not in _lib.DTYPE_CODE:
            raise RuntimeError("clip_grad_norm: gradients must be CUDA float32, bfloat16 or float16 tensors")
        if any(g.dtype != g0.dtype for g in grads):
            # several dtypes (float32 embeddings beside a bfloat16 body): per-dtype passes, norms combined in float32
            if torch.cuda.is_current_stream_capturing():
                raise NotImplementedError("clip_grad_norm over several dtypes cannot be captured into a CUDA graph")
            with_grad = [p for group in self.param_groups for p in group["params"] if p.grad is not None]
            return self._clip_from_sumsq(with_grad, list(range(len(with_grad))), [p.grad.dtype for p in with_grad], max_norm)
        for g in grads:
            if g.device != g0.device:
                raise NotImplementedError("clip_grad_norm: all gradients must live on one device")
            if not g.is_contiguous() and not is_dense(g):
                raise RuntimeError("clip_grad_norm: gradients must be dense")
        if self._clip_out is None or self._clip_out.device != g0.device:
            self._clip_out = torch.zeros(2, dtype=torch.float32, device=g0.device)
        numels = _lib.numel_array(grads)
        numels_arg = ctypes.cast(numels, ctypes.c_void_p)
        need = _lib.LIB.optimi_b200_grad_clip_workspace_bytes(len(grads), numels_arg)
        stream_ptr = torch._C._cuda_getCurrentRawStream(g0.device.index)
        ws = F._stable_workspace(g0.device, stream_ptr, need)
        ptrs = _lib.PointerArray(grads)
        capturing = torch.cuda.is_current_stream_capturing()
        record = _lib.graph_record() if capturing else None  # nothing in these launches changes from step to step
        with torch.cuda.device(g0.device):
            if record is not None:
                record.__enter__()
            try:
                rc = _lib.LIB.optimi_b200_grad_clip_factor(len(grads), ptrs.ptr, numels_arg, _lib.DTYPE_CODE[g0.dtype], float(max_norm),
                                                           self._clip_out.data_ptr(), ws.data_ptr(), ws.numel(), stream_ptr)  # fmt: skip
            finally:
                if record is not None:
                    record.__exit__(None, None, None)
        _lib.check(rc)
        self._grad_factor, self._grad_factor_once = self._clip_out[:1], not capturing
        return self._clip_out[1].clone()  # the two-float buffer is reused by the next call

    def _index_tensor(self, indices: tuple, device: torch.device) -> Tensor:
        """A device tensor of `indices`, kept for the next call (the same few index sets recur every step)."""
        cache = self.__dict__.setdefault("_index_tensors", {})
        t = cache.get((indices, device))
        if t is None:
            t = cache[(indices, device)] = torch.tensor(indices, dtype=torch.int64, device=device)
        return t

    @torch.no_grad()
    def _clip_from_sumsq(self, tensors: list[Tensor], owners: list[int], dtypes: list[torch.dtype], max_norm: float,
                         reduce_sums: Callable[[Tensor], None] | None = None) -> Tensor:  # fmt: skip
        """The clip coefficient in separable steps (the general form behind `clip_grad_norm`): `tensors` are
        parameters, or pieces of parameters, whose `.grad` is read; `owners[i]` is the index of the whole
        tensor that piece i belongs to and `dtypes[j]` the dtype of whole tensor j.  Per-piece sums of squares
        (double) are added into per-tensor sums, `reduce_sums` (if given) adds the other ranks' contributions
        in place, each tensor's norm is rounded to its own dtype as `torch._foreach_norm` would return it, and
        the coefficient is computed in the dtype PyTorch promotes the stacked norms to (the common dtype, or
        float32 when they differ).  Arms the next `step()` with the coefficient; returns the total norm."""
        device = None
        for t in tensors:
            if t.grad is not None:
                device = t.grad.device
                break
        if device is None:
            device = tensors[0].device if tensors else torch.device("cuda", torch.cuda.current_device())
        n_full = len(dtypes)
        sumsq = torch.zeros(n_full, dtype=torch.float64, device=device)
        stream_ptr = torch._C._cuda_getCurrentRawStream(device.index)
        by_dtype: dict[torch.dtype, list[int]] = {}
        for i, t in enumerate(tensors):
            if t.grad is None:
                continue
            g = t.grad
            if not g.is_cuda or g.dtype not in _lib.DTYPE_CODE or g.device != device:
                raise RuntimeError("clip_grad_norm: gradients must be CUDA float32, bfloat16 or float16 tensors on one device")
            if not g.is_contiguous() and not is_dense(g):
                raise RuntimeError("clip_grad_norm: gradients must be dense")
            by_dtype.setdefault(g.dtype, []).append(i)
        with torch.cuda.device(device):
            for dtype, idx in by_dtype.items():
                grads = [tensors[i].grad for i in idx]
                numels = _lib.numel_array(grads)
                numels_arg = ctypes.cast(numels, ctypes.c_void_p)
                need = _lib.LIB.optimi_b200_grad_clip_workspace_bytes(len(grads), numels_arg)
                ws = F._stable_workspace(device, stream_ptr, need)
                piece = torch.empty(len(grads), dtype=torch.float64, device=device)
                ptrs = _lib.PointerArray(grads)
                _lib.check(_lib.LIB.optimi_b200_grad_sumsq(len(grads), ptrs.ptr, numels_arg, _lib.DTYPE_CODE[dtype], piece.data_ptr(),
                                                          ws.data_ptr(), ws.numel(), stream_ptr))  # fmt: skip
                # a whole tensor has at most one piece in `tensors`, so this is a plain scatter
                sumsq[self._index_tensor(tuple(owners[i] for i in idx), device)] = piece
            if reduce_sums is not None:
                reduce_sums(sumsq)
            norms = torch.zeros(n_full, dtype=torch.float32, device=device)
            kinds = sorted(set(dtypes), key=str)
            for dtype in kinds:
                sel = self._index_tensor(tuple(j for j, d in enumerate(dtypes) if d == dtype), device)
                sub = sumsq[sel].contiguous()
                out = torch.empty(sub.numel(), dtype=torch.float32, device=device)
                _lib.check(_lib.LIB.optimi_b200_grad_norms_from_sumsq(sub.numel(), sub.data_ptr(), _lib.DTYPE_CODE[dtype], out.data_ptr(), stream_ptr))
                norms[sel] = out
            total_dtype = kinds[0] if len(kinds) == 1 else torch.float32
            if self._clip_out is None or self._clip_out.device != device:
                self._clip_out = torch.zeros(2, dtype=torch.float32, device=device)
            _lib.check(_lib.LIB.optimi_b200_clip_factor_from_norms(n_full, norms.data_ptr(), _lib.DTYPE_CODE[total_dtype], float(max_norm),
                                                                   self._clip_out.data_ptr(), stream_ptr))  # fmt: skip
        self._grad_factor, self._grad_factor_once = self._clip_out[:1], True
        return self._clip_out[1].clone()

    # ---- the step inside a CUDA graph -----------------------------------------------------------
    def _capture_step(self) -> None:
        """`step()` on a capturing stream: the launches go into the graph and the library remembers
        which nodes they became.  Nothing runs and no step counter moves; `update_graph` gives the
        nodes the scalars of each coming step."""
        record = _lib.graph_record()
        with record:
            for group in self.param_groups:
                self._step_group(group, capturing=True)
        self._graph_nodes = record.nodes

    def update_graph(self, graph: "torch.cuda.CUDAGraph") -> None:
        """Prepares the next replay of a CUDA graph that holds a captured `step()`.

        The kernels take the step's host scalars (bias corrections from the step count, the current
        `lr` and the other hyper-parameters of each `param_group`, Ranger's lookahead flag) by value,
        so a captured step has to be told about every new step: this advances the step counters as
        `step()` would and rewrites the kernel parameters of the captured launches in the
        instantiated graph, without launching anything.  Call it once before every
        `graph.replay()`.  The graph must have been created with `keep_graph=True` and instantiated
        (`torch.cuda.CUDAGraph(keep_graph=True)`, capture, `graph.instantiate()`): updating an
        instantiated graph names its nodes through the captured graph, which PyTorch otherwise
        discards.  Optimizer states must exist before the capture (run one eager step first) and
        gradients have to live where they lived during capture or be re-pointed before this call,
        which also passes the current gradient addresses on.

            opt.step()                                   # eager: creates the states
            g = torch.cuda.CUDAGraph(keep_graph=True)
            with torch.cuda.graph(g):
                opt.step()                               # captured, not run
            g.instantiate()
            for _ in range(steps):
                ...fill the static gradients, change param_group["lr"]...
                opt.update_graph(g)
                g.replay()
        """
        if self._graph_nodes is None:
            raise RuntimeError("update_graph: no captured step to update; call step() under torch.cuda.graph(...) first")
        graph.raw_cuda_graph()  # raises unless the graph was created with keep_graph=True
        graph_exec = graph.raw_cuda_graph_exec()
        factor = self._grad_factor
        if factor is not None:
            _lib.LIB.optimi_b200_grad_scale_begin(factor.data_ptr())
        try:
            with torch.no_grad(), _lib.graph_update(self._graph_nodes, graph_exec):
                for group in self.param_groups:
                    self._step_group(group)
        finally:
            if factor is not None:
                _lib.LIB.optimi_b200_grad_scale_end()
                if self._grad_factor_once:  # an eager clip_grad_norm() before this replay: its coefficient is for this step only
                    self._grad_factor = None

    # ---- whole-list step of one parameter group ---------------------------------------------------
    def _step_group(self, group: dict[str, Any], capturing: bool = False) -> None:
        """One step of every parameter of `group` that has a gradient: one C call per (device, dtype).

        The pointer tables of parameters and states are cached (`_GroupPlan`) for as long as the same
        parameters have gradients and nothing moved; a step then only re-reads the gradient
        addresses, re-checks the cached ones and calls the entry point, about a third of a
        millisecond of host time for 300 tensors instead of one and a half.
        """
        params = [p for p in group["params"] if p.grad is not None]
        key = tuple(map(id, params))
        plan = self._group_plans.get(id(group))
        if plan is None or plan.key != key or not plan.fresh():
            if capturing and (not group["setup"] or any("kahan_comp" not in self.state[p] for p in params)):
                raise RuntimeError(
                    "step() under CUDA graph capture needs the optimizer states to exist already (their allocation and "
                    "zero-fill would become part of the graph): run one eager step() before capturing"
                )
            for p in params:
                self._init_state(group, self.state[p], p)
            self._setup_group(group)
            plan = self._group_plans[id(group)] = _GroupPlan(self, group, params, key) if params else None
        t = 0
        if self._counts_steps:
            if capturing:  # nothing runs during capture: the counter moves in update_graph
                t = int(group["step"].item()) + 1
            else:
                t = F._advance(group["step"])  # the reference advances the counter even when no parameter has a gradient
        if plan is None:
            return
        tail = type(self)._tail(t, True, kahan_sum=group["kahan_sum"], **{k: group[k] for k in self._scalar_keys})
        for sub in plan.subs:
            sub.launch(tail, self._needs_workspace)

    # ---- gradient release: the per-parameter step ------------------------------------------------
    def _release(self, param: Tensor) -> None:
        """Steps one parameter from its gradient (the body of `step(param=...)` and of the hook).

        This runs once per parameter per backward pass on the autograd thread, where every
        microsecond delays the enqueueing of the backward pass itself, so it is kept lean: the
        C arguments are prebuilt per parameter (`_ReleasePlan`), the host scalars are computed once
        per (group, step count) and shared by the group's parameters, the step counter tensor is
        advanced through a numpy view, and the launch goes straight to the C entry point.
        Semantics are those of the reference's `step(param=...)` (optimi/adam.py:183-208): lazy state
        creation, a per-parameter step counter that also advances on accumulation micro-steps.
        """
        plan = self._plans.get(param)
        if plan is None or not plan.fresh(param):
            plan = self._plans[param] = self._make_plan(param)
        grad = param.grad
        if grad.dtype != param.dtype or not _dense_like(grad, param):
            raise RuntimeError(f"{plan.fn_name}: the gradient does not match its parameter's dtype or layout")
        plan.grad_slot[0] = grad.data_ptr()

        t = 0
        if plan.step_view is not None:
            plan.step_view += 1
            t = int(plan.step_view)
        update = not self._optimizer_accumulation
        group = plan.group
        key = (t, update, group["kahan_sum"], *[group[k] for k in self._scalar_keys])
        cached = self._tail_cache.get(id(group))
        if cached is not None and cached[0] == key:
            tail = cached[1]
        else:
            tail = type(self)._tail(t, update, kahan_sum=group["kahan_sum"], **{k: group[k] for k in self._scalar_keys})
            self._tail_cache[id(group)] = (key, tail)

        side = self._enter_release_stream(param)
        stream_ptr = side.cuda_stream if side is not None else torch._C._cuda_getCurrentRawStream(plan.index)
        if self._needs_workspace:
            tail = tail + (F.stable_workspace_args(plan.device, stream_ptr, (param,)) if update else (None, 0))
        factor = self._grad_factor
        if factor is not None:
            _lib.LIB.optimi_b200_grad_scale_begin(factor.data_ptr())
        if torch._C._cuda_getDevice() == plan.index:
            rc = plan.fn(1, *plan.args, plan.numels_arg, plan.dtype_code, *tail, stream_ptr)
        else:
            with torch.cuda.device(plan.device):
                rc = plan.fn(1, *plan.args, plan.numels_arg, plan.dtype_code, *tail, stream_ptr)
        if factor is not None:
            _lib.LIB.optimi_b200_grad_scale_end()
        if rc != 0:
            _lib.check(rc)
        if side is not None:
            grad.record_stream(side)

    def _make_plan(self, param: Tensor) -> "_ReleasePlan":
        state = self.state[param]
        group = state["group"]
        with torch.no_grad():
            self._init_state(group, state, param)
        if not param.is_cuda:
            raise RuntimeError(f"{self._c_fn}: parameters live on {param.device}; optimi_b200 steps CUDA tensors only (there is no CPU path)")
        if param.dtype not in _lib.DTYPE_CODE:
            raise RuntimeError(f"{self._c_fn}: unsupported parameter dtype {param.dtype} (float32, bfloat16 and float16 are)")
        return _ReleasePlan(self._c_fn, param, group, [state[k] for k in self._c_states], state.get("step") if self._counts_steps else None)

    # ---- gradient release on a side stream ----------------------------------------------------
    def use_release_stream(self, stream: torch.cuda.Stream | bool | None = True) -> None:
        """Runs the per-parameter steps of gradient release on a side stream so that they overlap
        with the rest of the backward pass (`prepare_for_gradient_release` switches this on by default for
        CUDA models).  `True` creates a stream, `None`/`False` goes back to stepping on the stream the hook
        fires on (the reference's behaviour).

        Ordering: each step waits for the gradient it consumes; the stream that runs the backward
        pass waits for all side-stream steps when the backward pass ends, so code after
        `loss.backward()` sees updated parameters without further synchronisation.
        """
        if stream is True:
            stream = torch.cuda.Stream()
        self._release_stream = stream or None
        self._release_stream_chosen = True

    def _enter_release_stream(self, param: Tensor):
        side = self._release_stream
        if side is None:
            return None
        main = torch.cuda.current_stream(param.device)
        side.wait_stream(main)
        if not self._release_fence_queued:
            self._release_fence_queued = True

            def fence():
                self._release_fence_queued = False
                main.wait_stream(side)

            try:
                torch.autograd.Variable._execution_engine.queue_callback(fence)
            except RuntimeError:
                # not inside a backward pass (a manual step(param=...) call): fence right away
                self._release_fence_queued = False
                return None
        return side

    @torch._disable_dynamo
    def zero_grad(self, set_to_none: bool = True, param: Tensor | None = None):
        """Resets the gradients of all optimized parameters, or of `param` alone (gradient release)."""
        if param is None:
            super().zero_grad(set_to_none=set_to_none)
        elif param.grad is not None:
            if set_to_none:
                param.grad = None
            else:
                if param.grad.grad_fn is not None:
                    param.grad.detach_()
                else:
                    param.grad.requires_grad_(False)


def _defaults(**kw) -> dict[str, Any]:
    kw["setup"] = False
    return kw


class Adam(OptimiOptimizer):
    """Adam optimizer, optionally with decoupled weight decay (AdamW).

    Same arguments as the reference (optimi/adam.py:56-70): `params`, `lr`, `betas=(0.9, 0.99)`,
    `weight_decay=0` (L2 unless `decouple_wd`/`decouple_lr`), `eps=1e-6`, `decouple_wd=False`,
    `decouple_lr=False`, `max_lr=None`, `kahan_sum=None` (auto: on for bf16/fp16 parameters),
    `foreach=None` and `triton=None` (accepted, ignored), `gradient_release=False`.
    """

    _c_fn, _c_states, _tail = "optimi_b200_adam", ("exp_avg", "exp_avg_sq", "kahan_comp"), staticmethod(T.adam_tail)
    _scalar_keys = ("lr", "beta1", "beta2", "weight_decay", "eps", "decouple_wd", "decouple_lr", "max_lr")

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 0,
        eps: float = 1e-6,
        decouple_wd: bool = False,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        kahan_sum: bool | None = None,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        _check_range("beta1", betas[0], "betas[0]")
        _check_range("beta2", betas[1], "betas[1]")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon: {eps=}")
        super().__init__(params, _defaults(
            lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay, decouple_wd=decouple_wd,
            decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum, foreach=foreach, triton=triton,
            gradient_release=gradient_release,
        ))  # fmt: skip

    def _new_state(self, group, state, param):
        state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)


class AdamW(Adam):
    """AdamW: Adam with decoupled weight decay, `weight_decay=1e-2` by default (optimi/adamw.py:48-75)."""

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 1e-2,
        eps: float = 1e-6,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        kahan_sum: bool | None = None,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        super().__init__(
            params=params, lr=lr, betas=betas, weight_decay=weight_decay, eps=eps, decouple_wd=True, decouple_lr=decouple_lr,
            max_lr=max_lr, kahan_sum=kahan_sum, foreach=foreach, triton=triton, gradient_release=gradient_release,
        )  # fmt: skip


class RAdam(Adam):
    """Rectified Adam (optimi/radam.py:57-71); same arguments as `Adam`."""

    _c_fn, _tail = "optimi_b200_radam", staticmethod(T.radam_tail)


class Ranger(OptimiOptimizer):
    """Ranger: RAdam plus Lookahead every `k` steps with step size `alpha` (optimi/ranger.py:59-75).
    Weight decay is decoupled by default."""

    _c_fn, _c_states, _tail = "optimi_b200_ranger", ("exp_avg", "exp_avg_sq", "la_param", "kahan_comp"), staticmethod(T.ranger_tail)
    _scalar_keys = ("lr", "beta1", "beta2", "weight_decay", "eps", "k", "alpha", "decouple_wd", "decouple_lr", "max_lr")

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 0,
        eps: float = 1e-6,
        k: int = 6,
        alpha: float = 0.5,
        decouple_wd: bool = True,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        kahan_sum: bool | None = None,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        _check_range("beta1", betas[0], "betas[0]")
        _check_range("beta2", betas[1], "betas[1]")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon: {eps=}")
        super().__init__(params, _defaults(
            lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay, k=k, alpha=alpha,
            decouple_wd=decouple_wd, decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum, foreach=foreach,
            triton=triton, gradient_release=gradient_release,
        ))  # fmt: skip

    def _new_state(self, group, state, param):
        state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        state["la_param"] = param.data.clone()


class Lion(OptimiOptimizer):
    """Lion, evolved sign momentum (optimi/lion.py:56-68).  Weight decay is always decoupled."""

    _c_fn, _c_states, _tail = "optimi_b200_lion", ("exp_avg", "kahan_comp"), staticmethod(T.lion_tail)
    _counts_steps = False
    _scalar_keys = ("lr", "beta1", "beta2", "weight_decay", "decouple_lr", "max_lr")

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 0,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        kahan_sum: bool | None = None,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        _check_range("beta1", betas[0], "betas[0]")
        _check_range("beta2", betas[1], "betas[1]")
        super().__init__(params, _defaults(
            lr=lr, beta1=betas[0], beta2=betas[1], weight_decay=weight_decay, decouple_lr=decouple_lr, max_lr=max_lr,
            kahan_sum=kahan_sum, foreach=foreach, triton=triton, gradient_release=gradient_release,
        ))  # fmt: skip

    def _new_state(self, group, state, param):
        state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)


class SGD(OptimiOptimizer):
    """SGD with optional momentum, dampening and (decoupled) weight decay (optimi/sgd.py:63-78).
    `torch_init=True` seeds the momentum buffer with the first gradient when dampening."""

    _c_fn, _c_states, _tail = "optimi_b200_sgd", ("exp_avg", "kahan_comp"), staticmethod(T.sgd_tail)
    _counts_steps = False
    _scalar_keys = ("lr", "momentum", "weight_decay", "dampening", "decouple_wd", "decouple_lr", "max_lr")

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        momentum: float = 0,
        weight_decay: float = 0,
        dampening: bool = False,
        decouple_wd: bool = False,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        torch_init: bool = False,
        kahan_sum: bool | None = None,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        if not 0.0 <= momentum < 1.0:
            raise ValueError(f"Invalid momentum: {momentum=}")
        super().__init__(params, _defaults(
            lr=lr, momentum=momentum, weight_decay=weight_decay, dampening=dampening, decouple_wd=decouple_wd,
            decouple_lr=decouple_lr, max_lr=max_lr, kahan_sum=kahan_sum, torch_init=torch_init, foreach=foreach,
            triton=triton, gradient_release=gradient_release,
        ))  # fmt: skip

    def _state_needs_first_gradient(self, group):
        return bool(group["dampening"] and group["torch_init"])

    def _new_state(self, group, state, param):
        if group["dampening"] and group["torch_init"]:
            # torch.optim.SGD seeds the buffer with the gradient after L2 decay (optimi/sgd.py:101-105)
            state["exp_avg"] = self._first_gradient(param)
            if group["weight_decay"] != 0 and not group["decouple_lr"] and not group["decouple_wd"]:
                state["exp_avg"].add_(param, alpha=group["weight_decay"])
        elif group["momentum"] != 0:
            state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        else:
            state["exp_avg"] = None


class StableAdamW(OptimiOptimizer):
    """StableAdamW: AdamW whose learning rate is clipped per tensor by the RMS of g^2/v
    (optimi/stableadamw.py:76-89).  The RMS is reduced on the device; a step never synchronises."""

    _c_fn, _c_states, _tail = "optimi_b200_stableadamw", ("exp_avg", "exp_avg_sq", "kahan_comp"), staticmethod(T.stableadamw_tail)
    _needs_workspace = True
    _scalar_keys = ("lr", "beta1", "beta2", "weight_decay", "eps", "decouple_lr", "max_lr")

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 1e-2,
        eps: float = 1e-6,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        kahan_sum: bool | None = None,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        _check_range("beta1", betas[0], "betas[0]")
        _check_range("beta2", betas[1], "betas[1]")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon: {eps=}")
        super().__init__(params, _defaults(
            lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay, decouple_lr=decouple_lr,
            max_lr=max_lr, kahan_sum=kahan_sum, foreach=foreach, triton=triton, gradient_release=gradient_release,
        ))  # fmt: skip

    def _new_state(self, group, state, param):
        state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        # kept for checkpoint compatibility with the reference (optimi/stableadamw.py:119)
        state["eps_sq"] = torch.tensor(group["eps"] ** 2, dtype=param.dtype, device=param.device)


class Adan(OptimiOptimizer):
    """Adan, adaptive Nesterov momentum (optimi/adan.py:62-76).  `kahan_sum` defaults to False here,
    unlike the other optimizers, and the class always applies Adan-style weight decay: like the
    reference it does not forward `adam_wd` to the functional step (optimi/adan.py:181-231)."""

    _c_fn, _c_states, _tail = ("optimi_b200_adan", ("exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp"),
                               staticmethod(T.adan_tail))  # fmt: skip
    _scalar_keys = ("lr", "beta1", "beta2", "beta3", "weight_decay", "eps", "decouple_lr", "max_lr")

    def __init__(
        self,
        params: Iterable[Tensor] | Iterable[dict],
        lr: float,
        betas: tuple[float, float, float] = (0.98, 0.92, 0.99),
        weight_decay: float = 2e-2,
        eps: float = 1e-6,
        decouple_lr: bool = False,
        max_lr: float | None = None,
        adam_wd: bool = False,
        kahan_sum: bool | None = False,
        foreach: bool | None = None,
        triton: bool | None = None,
        gradient_release: bool = False,
    ):
        _check_range("beta1", betas[0], "betas[0]")
        _check_range("beta2", betas[1], "betas[1]")
        _check_range("beta3", betas[2], "betas[2]")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon: {eps=}")
        super().__init__(params, _defaults(
            lr=lr, beta1=betas[0], beta2=betas[1], beta3=betas[2], eps=eps, weight_decay=weight_decay,
            decouple_lr=decouple_lr, max_lr=max_lr, adam_wd=adam_wd, kahan_sum=kahan_sum, foreach=foreach, triton=triton,
            gradient_release=gradient_release,
        ))  # fmt: skip

    def _state_needs_first_gradient(self, group):
        return True

    def _new_state(self, group, state, param):
        state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        state["exp_avg_diff"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)
        # negated first gradient, so the first gradient difference is zero (optimi/adan.py:109)
        state["prev_grad"] = self._first_gradient(param).mul_(-1)

    def _setup_group(self, group):
        first = not group["setup"]
        super()._setup_group(group)
        if first and group["kahan_sum"]:
            group["adam_wd"] = False  # optimi/adan.py:156-157
