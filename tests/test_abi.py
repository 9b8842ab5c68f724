"""The C-ABI library loads without a GPU, exports every symbol the header declares, and rejects bad
arguments before touching the device."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "optimi_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(optimi_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from optimi_b200 import _lib

    syms = declared_symbols()
    assert len(syms) >= 11, syms
    for name in syms:
        assert hasattr(_lib.LIB, name), f"{name} declared in include/optimi_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == syms
    assert _lib.LIB.optimi_b200_version() >= 100


def test_invalid_arguments_are_reported_not_launched():
    from optimi_b200 import _lib

    L = _lib.LIB
    before = L.optimi_b200_launch_count()
    nul = ctypes.c_void_p(0)
    one = (ctypes.c_int64 * 1)(16)
    numels = ctypes.cast(one, ctypes.c_void_p)
    # negative tensor count
    rc = L.optimi_b200_adam(-1, nul, nul, nul, nul, nul, nul, 1, 1e-3, 0.1, 0.99, 0.01, 0.0, 1e-6, 0, 1, 1, nul)
    assert rc == -1 and b"negative" in L.optimi_b200_last_error()
    # unknown dtype
    rc = L.optimi_b200_lion(1, nul, nul, nul, nul, numels, 7, 1e-4, 0.1, 0.01, 0.0, 0, 1, nul)
    assert rc == -1 and b"dtype" in L.optimi_b200_last_error()
    # a required list missing
    rc = L.optimi_b200_sgd(1, nul, nul, nul, nul, numels, 1, 1e-2, 0.9, 0.0, 0, 0, 0, 1, nul)
    assert rc == -1 and b"NULL" in L.optimi_b200_last_error()
    # a NULL tensor pointer inside a list
    arr = (ctypes.c_void_p * 1)(None)
    lst = ctypes.cast(arr, ctypes.c_void_p)
    rc = L.optimi_b200_adan(1, lst, lst, lst, lst, lst, lst, nul, numels, 0, 1e-3, 0.1, 0.92, 0.1, 0.99, 0.01, 1e-6, 0.0, 0, 0, 1, nul)
    assert rc == -1 and b"NULL pointer" in L.optimi_b200_last_error()
    # zero tensors is a no-op
    assert L.optimi_b200_radam(0, nul, nul, nul, nul, nul, nul, 1, 1e-3, 0.1, 0.99, 0.01, 0.0, 1e-6, 0, 0.0, 0, 0, 1, nul) == 0
    assert L.optimi_b200_launch_count() == before


def test_stableadamw_workspace_size_grows_with_the_list():
    from optimi_b200 import _lib

    small = (ctypes.c_int64 * 2)(1000, 5000)
    big = (ctypes.c_int64 * 2)(1000, 50_000_000)
    f = _lib.LIB.optimi_b200_stableadamw_workspace_bytes
    a = f(2, ctypes.cast(small, ctypes.c_void_p))
    b = f(2, ctypes.cast(big, ctypes.c_void_p))
    assert 16 <= a < b
    assert b >= 50_000_000 // 2048 * 8


def test_cpu_tensors_are_refused_loudly():
    import torch

    import optimi_b200

    p = torch.nn.Parameter(torch.zeros(8))
    p.grad = torch.ones(8)
    opt = optimi_b200.Lion([p], lr=1e-4)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        opt.step()


def test_graph_brackets_reject_misuse_without_touching_the_device():
    from optimi_b200 import _lib

    L = _lib.LIB
    assert L.optimi_b200_graph_record_end(None) == -1 and b"no record bracket" in L.optimi_b200_last_error()
    assert L.optimi_b200_graph_update_end() == -1 and b"no update bracket" in L.optimi_b200_last_error()
    assert L.optimi_b200_graph_update_begin(None, None) == -1 and b"nodes is NULL" in L.optimi_b200_last_error()
    assert L.optimi_b200_graph_record_begin() == 0
    assert L.optimi_b200_graph_record_begin() == -1 and b"already open" in L.optimi_b200_last_error()
    out = ctypes.c_void_p()
    assert L.optimi_b200_graph_record_end(ctypes.byref(out)) == 0 and out.value
    assert L.optimi_b200_graph_nodes_count(out) == 0  # a step with no launches
    assert L.optimi_b200_graph_update_begin(out, None) == -1 and b"graph_exec is NULL" in L.optimi_b200_last_error()
    L.optimi_b200_graph_nodes_free(out)
    L.optimi_b200_graph_nodes_free(None)


def test_grad_clip_factor_checks_its_arguments():
    from optimi_b200 import _lib

    L = _lib.LIB
    before = L.optimi_b200_launch_count()
    one = (ctypes.c_int64 * 1)(4096)
    numels = ctypes.cast(one, ctypes.c_void_p)
    arr = (ctypes.c_void_p * 1)(0x1000)
    lst = ctypes.cast(arr, ctypes.c_void_p)
    need = L.optimi_b200_grad_clip_workspace_bytes(1, numels)
    big = (ctypes.c_int64 * 1)(1 << 30)
    assert 32 <= need < L.optimi_b200_grad_clip_workspace_bytes(1, ctypes.cast(big, ctypes.c_void_p))
    fake = ctypes.c_void_p(0x2000)
    assert L.optimi_b200_grad_clip_factor(1, lst, numels, 1, 1.0, None, fake, need, None) == -1
    assert b"out is NULL" in L.optimi_b200_last_error()
    assert L.optimi_b200_grad_clip_factor(1, lst, numels, 1, 1.0, fake, fake, 8, None) == -3
    assert b"workspace" in L.optimi_b200_last_error()
    assert L.optimi_b200_grad_clip_factor(1, None, numels, 1, 1.0, fake, fake, need, None) == -1
    assert L.optimi_b200_launch_count() == before
