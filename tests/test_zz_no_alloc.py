"""StableAdamW through `optimi_b200_stableadamw_static`, the entry point for callers that cannot
allocate device memory.

Some users of the C ABI are handed the parameter, gradient and state pointers by a host runtime that
owns every byte of device memory and gives them no allocator (or they run where a cudaMalloc — which
synchronises the device and may fail under memory pressure — must not happen), so they have nothing to
pass as the `workspace` of `optimi_b200_stableadamw`.  The static variant keeps that scratch inside
the library.  This test drives both entry points through ctypes on identical inputs, twice in a row
(the second call reuses the scratch the first one left behind), and expects identical bits.

Collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.
"""

import ctypes

import pytest
import torch


def _ptrs(ts):
    return ctypes.cast((ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts]), ctypes.c_void_p), ts


def _call(static, tensors, dtype_code, kahan, lr, step, workspace=None):
    from optimi_b200 import _lib
    from optimi_b200.functional import debias_beta

    L = _lib.LIB
    p, g, m, v, k = tensors
    numels = (ctypes.c_int64 * len(p))(*[t.numel() for t in p])
    b1c = 1 - debias_beta(0.9, step)
    b2h = debias_beta(0.99, step)
    lists = [_ptrs(x)[0] for x in (p, g, m, v)] + [_ptrs(k)[0] if kahan else None]
    common = (len(p), *lists, ctypes.cast(numels, ctypes.c_void_p), dtype_code, lr, b1c, b2h, 1 - b2h, 1e-2, 1e-6, 0, 0.0,
              int(kahan), 1)  # fmt: skip
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if static:
        rc = L.optimi_b200_stableadamw_static(*common, stream)
    else:
        rc = L.optimi_b200_stableadamw(*common, ctypes.c_void_p(workspace.data_ptr()), workspace.numel(), stream)
    assert rc == 0, L.optimi_b200_last_error().decode()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,code,kahan", [(torch.bfloat16, 1, True), (torch.float32, 0, False)], ids=["bf16-kahan", "f32"])
def test_static_scratch_entry_matches_workspace_entry(dtype, code, kahan):
    from optimi_b200 import _lib

    gen = torch.Generator().manual_seed(7)
    shapes = [(513, 257), (4096,), (100_003,), (3,), (1 << 20,)]
    base = {
        "p": [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in shapes],
        "m": [torch.zeros(s, dtype=dtype) for s in shapes],
        "v": [torch.zeros(s, dtype=dtype) for s in shapes],
        "k": [torch.zeros(s, dtype=dtype) for s in shapes],
    }
    # the second tensor gets large gradients so that its learning rate is actually clipped
    grads = [[(torch.randn(s, generator=gen) * (5.0 if i == 1 else 1e-3)).to(dtype) for i, s in enumerate(shapes)] for _ in range(2)]

    def fresh():
        return [[t.clone().cuda() for t in base[name]] for name in ("p", "m", "v", "k")]

    (p1, m1, v1, k1), (p2, m2, v2, k2) = fresh(), fresh()
    numels = (ctypes.c_int64 * len(shapes))(*[t.numel() for t in p1])
    need = _lib.LIB.optimi_b200_stableadamw_workspace_bytes(len(shapes), ctypes.cast(numels, ctypes.c_void_p))
    workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    for step in (1, 2):  # two calls in a row: the static scratch still holds the first call's partial sums
        g1 = [g.clone().cuda() for g in grads[step - 1]]
        g2 = [g.clone().cuda() for g in grads[step - 1]]
        _call(False, (p1, g1, m1, v1, k1), code, kahan, 3e-4, step, workspace)
        _call(True, (p2, g2, m2, v2, k2), code, kahan, 3e-4, step)
        torch.cuda.synchronize()
        for name, a, b in (("param", p1, p2), ("exp_avg", m1, m2), ("exp_avg_sq", v1, v2), ("kahan_comp", k1, k2)):
            for i, (x, y) in enumerate(zip(a, b)):
                assert torch.equal(x, y), f"step {step}: {name}[{i}] differs between the two entry points"
    assert not torch.equal(p1[1].cpu(), base["p"][1])  # the step did something


def test_static_scratch_entry_rejects_lists_beyond_its_limit():
    """The size check comes before any CUDA call, so it is testable without a device: 2^32 fp32
    elements need 64 MiB of partial sums, the built-in scratch holds 4 MiB."""
    from optimi_b200 import _lib

    L = _lib.LIB
    before = L.optimi_b200_launch_count()
    fake = (ctypes.c_void_p * 1)(0x1000)  # never dereferenced: the call must fail before launching
    lst = ctypes.cast(fake, ctypes.c_void_p)
    numels = (ctypes.c_int64 * 1)(1 << 32)
    rc = L.optimi_b200_stableadamw_static(1, lst, lst, lst, lst, None, ctypes.cast(numels, ctypes.c_void_p), 0, 3e-4, 0.1, 0.99,
                                          0.01, 1e-2, 1e-6, 0, 0.0, 0, 1, None)  # fmt: skip
    assert rc == -3
    msg = L.optimi_b200_last_error().decode()
    assert "built-in scratch" in msg and "split the list" in msg
    assert L.optimi_b200_launch_count() == before
