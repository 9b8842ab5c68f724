"""ctypes binding of liboptimi_b200.so (the C ABI declared in include/optimi_b200.h).

There is no fallback: if the library cannot be loaded (and cannot be built because nvcc is absent)
importing this module raises, and a failing entry point raises ``RuntimeError`` with the library's
own message.
"""

from __future__ import annotations

import ctypes

import torch

from . import build as _build

OPTIMI_F32, OPTIMI_BF16, OPTIMI_F16 = 0, 1, 2
DTYPE_CODE = {torch.float32: OPTIMI_F32, torch.bfloat16: OPTIMI_BF16, torch.float16: OPTIMI_F16}

_P = ctypes.c_void_p  # host array of device pointers, or NULL
_D = ctypes.c_double
_I = ctypes.c_int

# name -> argument types after (n_tensors) and the pointer lists; mirrors include/optimi_b200.h
SIGNATURES = {
    "optimi_b200_adam": [_I] + [_P] * 5 + [_P, _I] + [_D] * 6 + [_I] * 3 + [_P],
    "optimi_b200_lion": [_I] + [_P] * 4 + [_P, _I] + [_D] * 4 + [_I] * 2 + [_P],
    "optimi_b200_sgd": [_I] + [_P] * 4 + [_P, _I] + [_D] * 3 + [_I] * 4 + [_P],
    "optimi_b200_stableadamw": [_I] + [_P] * 5 + [_P, _I] + [_D] * 6 + [_I, _D, _I, _I, _P, ctypes.c_size_t, _P],
    "optimi_b200_stableadamw_static": [_I] + [_P] * 5 + [_P, _I] + [_D] * 6 + [_I, _D, _I, _I, _P],
    "optimi_b200_adan": [_I] + [_P] * 7 + [_P, _I] + [_D] * 8 + [_I] * 3 + [_P],
    "optimi_b200_radam": [_I] + [_P] * 5 + [_P, _I] + [_D] * 6 + [_I, _D] + [_I] * 3 + [_P],
    "optimi_b200_ranger": [_I] + [_P] * 6 + [_P, _I] + [_D] * 6 + [_I, _D, _I, _D] + [_I] * 3 + [_P],
}
EXPORTS = list(SIGNATURES) + ["optimi_b200_push_begin", "optimi_b200_push_end", "optimi_b200_pull_begin", "optimi_b200_pull_end", "optimi_b200_last_error", "optimi_b200_version", "optimi_b200_launch_count", "optimi_b200_stableadamw_workspace_bytes",
                                   "optimi_b200_graph_record_begin", "optimi_b200_graph_record_end", "optimi_b200_graph_nodes_count",
                                   "optimi_b200_graph_nodes_free", "optimi_b200_graph_update_begin", "optimi_b200_graph_update_end",
                                   "optimi_b200_grad_scale_begin", "optimi_b200_grad_scale_end", "optimi_b200_grad_clip_workspace_bytes",
                                   "optimi_b200_grad_clip_factor", "optimi_b200_grad_sumsq", "optimi_b200_grad_norms_from_sumsq",
                                   "optimi_b200_clip_factor_from_norms"]  # fmt: skip


def _load() -> ctypes.CDLL:
    path = _build.LIB
    if not _build.up_to_date():
        # not built yet, or built from other sources: build now (needs nvcc), else fail loudly
        path = _build.build(force=True)
    lib = ctypes.CDLL(path)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _I
    lib.optimi_b200_last_error.restype = ctypes.c_char_p
    lib.optimi_b200_last_error.argtypes = []
    lib.optimi_b200_version.restype = _I
    lib.optimi_b200_push_begin.restype = _I
    lib.optimi_b200_push_begin.argtypes = [_I, _P]
    lib.optimi_b200_push_end.restype = None
    lib.optimi_b200_push_end.argtypes = []
    lib.optimi_b200_pull_begin.restype = _I
    lib.optimi_b200_pull_begin.argtypes = [_I, _P, _D]
    lib.optimi_b200_pull_end.restype = None
    lib.optimi_b200_pull_end.argtypes = []
    lib.optimi_b200_launch_count.restype = ctypes.c_ulonglong
    lib.optimi_b200_launch_count.argtypes = []
    lib.optimi_b200_stableadamw_workspace_bytes.restype = ctypes.c_size_t
    lib.optimi_b200_stableadamw_workspace_bytes.argtypes = [_I, _P]
    lib.optimi_b200_grad_scale_begin.restype = None
    lib.optimi_b200_grad_scale_begin.argtypes = [_P]
    lib.optimi_b200_grad_scale_end.restype = None
    lib.optimi_b200_grad_scale_end.argtypes = []
    lib.optimi_b200_grad_clip_workspace_bytes.restype = ctypes.c_size_t
    lib.optimi_b200_grad_clip_workspace_bytes.argtypes = [_I, _P]
    lib.optimi_b200_grad_clip_factor.restype = _I
    lib.optimi_b200_grad_clip_factor.argtypes = [_I, _P, _P, _I, _D, _P, _P, ctypes.c_size_t, _P]
    lib.optimi_b200_grad_sumsq.restype = _I
    lib.optimi_b200_grad_sumsq.argtypes = [_I, _P, _P, _I, _P, _P, ctypes.c_size_t, _P]
    lib.optimi_b200_grad_norms_from_sumsq.restype = _I
    lib.optimi_b200_grad_norms_from_sumsq.argtypes = [_I, _P, _I, _P, _P]
    lib.optimi_b200_clip_factor_from_norms.restype = _I
    lib.optimi_b200_clip_factor_from_norms.argtypes = [_I, _P, _I, _D, _P, _P]
    lib.optimi_b200_graph_record_begin.restype = _I
    lib.optimi_b200_graph_record_begin.argtypes = []
    lib.optimi_b200_graph_record_end.restype = _I
    lib.optimi_b200_graph_record_end.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
    lib.optimi_b200_graph_nodes_count.restype = _I
    lib.optimi_b200_graph_nodes_count.argtypes = [_P]
    lib.optimi_b200_graph_nodes_free.restype = None
    lib.optimi_b200_graph_nodes_free.argtypes = [_P]
    lib.optimi_b200_graph_update_begin.restype = _I
    lib.optimi_b200_graph_update_begin.argtypes = [_P, _P]
    lib.optimi_b200_graph_update_end.restype = _I
    lib.optimi_b200_graph_update_end.argtypes = []
    return lib


LIB = _load()
LIB_PATH = _build.LIB


class peer_push:
    """Context manager: launches made by this thread inside it also store updated parameters into the
    peers' copies of the parameter buffer (`deltas`: byte offsets to those copies)."""

    def __init__(self, deltas):
        self.deltas = (ctypes.c_int64 * len(deltas))(*deltas)

    def __enter__(self):
        check(LIB.optimi_b200_push_begin(len(self.deltas), ctypes.cast(self.deltas, ctypes.c_void_p)))
        return self

    def __exit__(self, *exc):
        LIB.optimi_b200_push_end()


class peer_pull:
    """Context manager: launches made by this thread inside it take as gradient the scaled fp32 sum of
    all ranks' gradient buffers (`deltas`: byte offsets to them in rank order, 0 for this rank)."""

    def __init__(self, deltas, scale: float):
        self.deltas, self.scale = (ctypes.c_int64 * len(deltas))(*deltas), scale

    def __enter__(self):
        check(LIB.optimi_b200_pull_begin(len(self.deltas), ctypes.cast(self.deltas, ctypes.c_void_p), self.scale))
        return self

    def __exit__(self, *exc):
        LIB.optimi_b200_pull_end()


class grad_scale:
    """Context manager: step launches made by this thread inside it multiply every gradient element by the
    fp32 value stored at `factor` (a CUDA float32 tensor with one element) as they load it."""

    def __init__(self, factor: torch.Tensor):
        if factor.dtype != torch.float32 or not factor.is_cuda or factor.numel() < 1:
            raise ValueError("the gradient factor must be a CUDA float32 tensor")
        self.factor = factor

    def __enter__(self):
        LIB.optimi_b200_grad_scale_begin(self.factor.data_ptr())
        return self

    def __exit__(self, *exc):
        LIB.optimi_b200_grad_scale_end()


class GraphNodes:
    """The CUDA-graph nodes that the launches of one captured step became (an owned C handle)."""

    def __init__(self, handle: int):
        self.handle = handle

    def __len__(self) -> int:
        return LIB.optimi_b200_graph_nodes_count(self.handle)

    def __del__(self):
        if self.handle and LIB is not None:
            LIB.optimi_b200_graph_nodes_free(self.handle)
            self.handle = None


class graph_record:
    """Context manager for a step made on a capturing stream: this thread's launches are captured as
    usual and their graph nodes remembered; `.nodes` holds them afterwards."""

    nodes: GraphNodes | None = None

    def __enter__(self):
        check(LIB.optimi_b200_graph_record_begin())
        return self

    def __exit__(self, *exc):
        out = ctypes.c_void_p()
        rc = LIB.optimi_b200_graph_record_end(ctypes.byref(out))
        if rc == 0:
            self.nodes = GraphNodes(out.value)
        if exc[0] is None:
            check(rc)


class graph_update:
    """Context manager: the step calls made by this thread inside it launch nothing; each would-be
    launch rewrites the kernel parameters of the corresponding recorded node in `graph_exec`."""

    def __init__(self, nodes: GraphNodes, graph_exec: int):
        self.nodes, self.graph_exec = nodes, graph_exec

    def __enter__(self):
        check(LIB.optimi_b200_graph_update_begin(self.nodes.handle, self.graph_exec))
        return self

    def __exit__(self, *exc):
        rc = LIB.optimi_b200_graph_update_end()
        if exc[0] is None:
            check(rc)


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"optimi_b200 (code {rc}): {LIB.optimi_b200_last_error().decode()}")


class PointerArray:
    """A host array of device pointers for one tensor list (kept alive for the duration of a call)."""

    __slots__ = ("arr",)

    def __init__(self, tensors):
        self.arr = (ctypes.c_void_p * len(tensors))(*map(torch.Tensor.data_ptr, tensors))

    @property
    def ptr(self):
        return ctypes.cast(self.arr, ctypes.c_void_p)


def pointer_list(tensors) -> PointerArray | None:
    return None if tensors is None else PointerArray(tensors)


def numel_array(tensors):
    return (ctypes.c_int64 * len(tensors))(*map(torch.Tensor.numel, tensors))
