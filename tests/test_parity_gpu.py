"""Parity of the CUDA kernels (through the classes and the C ABI) with the reference.

1. Every golden case (reference run on a B200) replayed through optimi_b200: bit-exact for all
   storage types, except
     - StableAdamW: the per-tensor mean is summed in a different (fixed) order than the reference's
       reduction, so float32 results agree to 1e-6 relative and 16-bit results to 1 ulp;
     - the Ranger bf16 gradient-release golden, which follows `_single_param_ranger`'s variant of
       the Kahan lookahead; the kernels follow the foreach/Triton variant and are checked
       against the oracle instead.
2. Larger seeded lists with ragged and misaligned tensors against the CPU oracle.
"""

import pytest
import torch

from cases import CASES, CASES_BY_NAME
from helpers import (TORCH_DTYPE, compare_exact, golden_tensor, load_golden, run_b200_case, run_oracle_case, ulp_diff,
                     within_ulps_of_scale)

pytestmark = pytest.mark.gpu

CUDA = load_golden("cuda")


def _check_stable(case, got, want_of):
    for key, t in got.items():
        w = want_of(key)
        t = t.detach().cpu().reshape(-1)
        w = w.reshape(-1)
        if case.dtype == "f32":
            ok = (t.double() - w.double()).abs() <= 1e-9 + 1e-6 * w.double().abs()
        else:
            ok = within_ulps_of_scale(t, w, 1.0, 1e-3)
        assert bool(ok.all()), f"{case.name} {key}: {int((~ok).sum())} elements off"


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_kernels_match_reference_golden(case):
    got = run_b200_case(case)
    want_of = lambda k: golden_tensor(CUDA, case, k)  # noqa: E731
    if case.opt == "stableadamw":
        _check_stable(case, got, want_of)
        return
    if case.name == "gr_ranger_bf16k_dwd":
        ref = run_oracle_case(case, single_param_lookahead=False)
        bad = compare_exact(got, lambda k: ref.get(k), case.name)
    else:
        bad = compare_exact(got, want_of, case.name)
    assert not bad, "\n".join(bad)


@pytest.mark.parametrize("name", ["gr_adam_bf16k_dwd", "gr_adan_bf16k_wd", "gr_stableadamw_bf16k_dwd", "gr_lion_f32_dwd"])
def test_release_stream_gives_same_result(name):
    case = CASES_BY_NAME[name]
    a = run_b200_case(case)
    b = run_b200_case(case, release_stream=True)
    for k in a:
        assert torch.equal(a[k], b[k]), k


# ----------------------------------------------------------------------------------------------
# bigger, ragged, misaligned lists against the oracle
# ----------------------------------------------------------------------------------------------
BIG_SHAPES = [(1 << 20) + 3, 65536, 4096, 4097, 1, 100_003, (300, 257), 8, 0, 16384 * 3 + 5]


def _big_inputs(dtype, seed, steps):
    g = torch.Generator().manual_seed(seed)
    params, grads = [], []
    for shp in BIG_SHAPES:
        shp = (shp,) if isinstance(shp, int) else shp
        params.append((torch.randn(shp, generator=g) * 0.02).to(dtype))
    scales = torch.exp(torch.randn(len(BIG_SHAPES), generator=g) + torch.log(torch.tensor(1e-3)))
    for _ in range(steps):
        grads.append([(torch.randn(p.shape, generator=g) * s).to(dtype) for p, s in zip(params, scales)])
    return params, grads


BIG = [
    ("adam", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True), "bf16"),
    ("adam", dict(lr=1e-3, weight_decay=1e-2), "f32"),
    ("adamw", dict(lr=3e-4), "f16"),
    ("lion", dict(lr=1e-4, weight_decay=0.1), "bf16"),
    ("sgd", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2), "bf16"),
    ("sgd", dict(lr=1e-2, momentum=0.9, dampening=True, torch_init=True, weight_decay=1e-2), "f32"),
    ("adan", dict(lr=3e-4, kahan_sum=True), "bf16"),
    ("adan", dict(lr=3e-4), "f32"),
    ("radam", dict(lr=3e-4, weight_decay=1e-2, decouple_wd=True), "bf16"),
    ("ranger", dict(lr=3e-4, weight_decay=1e-2, k=3), "bf16"),
    ("ranger", dict(lr=3e-4, k=3), "f32"),
    ("stableadamw", dict(lr=3e-4), "bf16"),
    ("stableadamw", dict(lr=3e-4), "f32"),
]


@pytest.mark.parametrize("opt,kw,dt", BIG, ids=[f"{o}-{d}-{i}" for i, (o, _, d) in enumerate(BIG)])
@pytest.mark.parametrize("misalign", [False, True], ids=["aligned", "misaligned"])
def test_kernels_match_oracle_on_ragged_lists(opt, kw, dt, misalign):
    import warnings

    import optimi_b200
    from cases import CLASS_NAMES, STATE_NAMES
    from oracle.port import OracleOptimizer

    dtype = TORCH_DTYPE[dt]
    steps = 7
    params, grads = _big_inputs(dtype, 1234, steps)
    oracle = OracleOptimizer(opt, [p.clone() for p in params], **kw)

    def dev(t):
        if not misalign:
            return t.cuda()
        # a view one element into a larger buffer: base address off the 16-byte grid
        buf = torch.empty(t.numel() + 1, dtype=t.dtype, device="cuda")
        v = buf[1:].view(t.shape)
        v.copy_(t)
        return v

    dparams = [dev(p).requires_grad_(True) for p in params]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt_gpu = getattr(optimi_b200, CLASS_NAMES[opt])(dparams, **kw)
    for it in range(steps):
        for p, g in zip(dparams, grads[it]):
            p.grad = dev(g)
        opt_gpu.step()
        opt_gpu.zero_grad()
        oracle.step([g.clone() for g in grads[it]])
    torch.cuda.synchronize()
    for i, p in enumerate(dparams):
        pairs = [("param", p.detach().cpu(), oracle.params[i])]
        for name in STATE_NAMES[opt]:
            t = opt_gpu.state[p].get(name)
            if t is not None and t.numel() == p.numel():
                pairs.append((name, t.cpu(), oracle.state[i][name]))
        for name, a, b in pairs:
            if a.numel() == 0:
                continue
            if opt == "stableadamw":
                if dt == "f32":
                    ok = (a.double() - b.double()).abs() <= 1e-9 + 1e-6 * b.double().abs()
                else:
                    ok = within_ulps_of_scale(a, b, 1.0, 1e-3)
                assert bool(ok.all()), f"tensor {i} {name}: {int((~ok).sum())} off"
            else:
                d = ulp_diff(a.reshape(-1), b.reshape(-1))
                assert int(d.max()) == 0, f"tensor {i} {name}: {int((d > 0).sum())}/{d.numel()} differ, max {int(d.max())} ulp"


FUNCTIONAL = [
    ("Adam", "adam", dict(lr=3e-4, weight_decay=1e-2), ("exp_avg", "exp_avg_sq", "kahan_comp")),
    ("AdamW", "adamw", dict(lr=3e-4, weight_decay=1e-5, decouple_lr=True), ("exp_avg", "exp_avg_sq", "kahan_comp")),
    ("Lion", "lion", dict(lr=1e-4, weight_decay=0.1), ("exp_avg", "kahan_comp")),
    ("SGD", "sgd", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2), ("exp_avg", "kahan_comp")),
    ("StableAdamW", "stableadamw", dict(lr=3e-4), ("exp_avg", "exp_avg_sq", "eps_sq", "kahan_comp")),
    ("Adan", "adan", dict(lr=3e-4, kahan_sum=True), ("exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp")),
    ("RAdam", "radam", dict(lr=3e-4), ("exp_avg", "exp_avg_sq", "kahan_comp")),
    ("Ranger", "ranger", dict(lr=3e-4, k=2), ("exp_avg", "exp_avg_sq", "la_param", "kahan_comp")),
]


@pytest.mark.parametrize("cname,fname,kw,keys", FUNCTIONAL, ids=[f[1] for f in FUNCTIONAL])
def test_functional_api_matches_classes(cname, fname, kw, keys):
    """The functional entry points (lists in, same keyword set as the reference's) and the classes are
    two doors to the same kernels: same inputs, same bits."""
    import warnings

    import optimi_b200

    gen = torch.Generator().manual_seed(5)
    shapes = [(257, 33), (4096,), (7,)]
    host = [(torch.randn(s, generator=gen) * 0.02).to(torch.bfloat16) for s in shapes]
    grads = [[(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16) for s in shapes] for _ in range(4)]
    a = [h.clone().cuda().requires_grad_(True) for h in host]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = getattr(optimi_b200, cname)(a, **kw)
    for gs in grads:
        for p, g in zip(a, gs):
            p.grad = g.cuda()
        opt.step()
    # functional: states start as the class creates them, hyper-parameters come from the class's group
    b = [h.clone().cuda() for h in host]
    group = opt.param_groups[0]
    fn = getattr(optimi_b200, fname)
    names = {"exp_avg": "exp_avgs", "exp_avg_sq": "exp_avg_sqs", "kahan_comp": "kahan_comps", "la_param": "la_params",
             "exp_avg_diff": "exp_avg_diffs", "prev_grad": "prev_grads", "eps_sq": "eps_sqs"}  # fmt: skip
    states = {}
    for k in keys:
        if k == "la_param":
            states[k] = [t.clone() for t in b]
        elif k == "prev_grad":
            states[k] = [-g.cuda() for g in grads[0]]
        elif k == "eps_sq":
            states[k] = [torch.tensor(group["eps"] ** 2, dtype=torch.bfloat16, device="cuda") for _ in b]
        elif k == "kahan_comp" and not group["kahan_sum"]:
            states[k] = None
        else:
            states[k] = [torch.zeros_like(t) for t in b]
    hyper = {k: v for k, v in group.items() if k not in ("params", "setup", "step", "foreach", "triton", "gradient_release", "torch_init")}
    if fname == "adamw":
        hyper.pop("decouple_wd")
    if fname == "adan":
        hyper.pop("adam_wd", None)
    step = torch.tensor(0, dtype=torch.int32)
    for gs in grads:
        kwargs = dict(hyper)
        if fname not in ("lion", "sgd"):
            kwargs["step"] = step
        fn(b, [g.cuda() for g in gs], **{names[k]: v for k, v in states.items()}, **kwargs)
    torch.cuda.synchronize()
    for i, (p, q) in enumerate(zip(a, b)):
        assert torch.equal(p.detach(), q), f"param {i}"
        for k in keys:
            if k in ("eps_sq",) or states[k] is None:
                continue
            assert torch.equal(opt.state[p][k], states[k][i]), f"{k} of tensor {i}"


def test_config1_full_size():
    """BASELINE configuration 1 at full size: kernels == oracle on every element (float32, bit for bit),
    and == the reference's CUDA foreach result on the sampled elements of the golden (when the golden
    file carries them)."""
    import optimi_b200
    from cases import CONFIG1_HYPER, CONFIG1_STRIDE, config1_grads, config1_params
    from oracle.port import OracleOptimizer

    host = [torch.from_numpy(p) for p in config1_params()]
    oracle = OracleOptimizer("adamw", [h.clone() for h in host], **CONFIG1_HYPER)
    params = [h.clone().cuda().requires_grad_(True) for h in host]
    opt = optimi_b200.AdamW(params, **CONFIG1_HYPER)
    for grads in config1_grads():
        gs = [torch.from_numpy(g) for g in grads]
        for p, g in zip(params, gs):
            p.grad = g.cuda()
        opt.step()
        opt.zero_grad()
        oracle.step(gs)
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        for name, got, want in (("param", p.detach(), oracle.params[i]), ("exp_avg", opt.state[p]["exp_avg"], oracle.state[i]["exp_avg"]),
                                ("exp_avg_sq", opt.state[p]["exp_avg_sq"], oracle.state[i]["exp_avg_sq"])):  # fmt: skip
            assert torch.equal(got.cpu(), want), f"tensor {i} {name} differs from the oracle"
            key = f"config1/{i}.{name}"
            if key in CUDA.files:
                assert torch.equal(got.cpu().reshape(-1)[::CONFIG1_STRIDE], torch.from_numpy(CUDA[key].copy())), f"tensor {i} {name} differs from the reference"


def test_permuted_dense_parameter_steps_like_its_memory():
    """The kernels pair elements by position in memory, so a dense but permuted parameter (a transposed view, a
    channels_last weight) whose gradient and states share its strides must end up exactly like the same memory
    stepped as a contiguous tensor; a gradient with other strides is refused."""
    import optimi_b200

    gen = torch.Generator().manual_seed(0)
    base = (torch.randn(64, 48, generator=gen) * 0.02).to(torch.bfloat16).cuda()
    grads = [(torch.randn(64, 48, generator=gen) * 1e-3).to(torch.bfloat16).cuda() for _ in range(3)]
    p = torch.nn.Parameter(base.clone().t())  # 48 x 64 with strides (1, 48): dense, not contiguous
    q = torch.nn.Parameter(base.clone())
    assert not p.is_contiguous()
    kw = dict(lr=1e-3, weight_decay=1e-2)
    a, b = optimi_b200.AdamW([p], **kw), optimi_b200.AdamW([q], **kw)
    for g in grads:
        p.grad, q.grad = g.t(), g
        a.step()
        b.step()
    torch.cuda.synchronize()
    assert torch.equal(p.detach().t(), q.detach())
    assert torch.equal(a.state[p]["exp_avg_sq"].t(), b.state[q]["exp_avg_sq"])
    p.grad = grads[0].t().contiguous()  # same shape, other strides
    with pytest.raises(RuntimeError, match="does not match its parameter"):
        a.step()


def test_step_groups_in_any_order_equals_one_step():
    """`step_groups` steps some parameter groups now and others later (each group has its own step counter); over
    all groups it must leave exactly what one `step()` leaves, whatever the order."""
    import optimi_b200

    gen = torch.Generator().manual_seed(4)
    shapes = [(257, 129), (4096,), (1000, 33), (7,)]
    host = [(torch.randn(s, generator=gen) * 0.02).to(torch.bfloat16) for s in shapes]

    def groups(ps):
        return [{"params": ps[:1]}, {"params": ps[1:3], "weight_decay": 0.0, "lr": 1e-3}, {"params": ps[3:]}]

    a = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    b = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    kw = dict(lr=3e-4, weight_decay=1e-2)
    whole, pieces = optimi_b200.AdamW(groups(a), **kw), optimi_b200.AdamW(groups(b), **kw)
    for it in range(4):
        for p, q in zip(a, b):
            g = (torch.randn(p.shape, generator=gen) * 1e-3).to(torch.bfloat16).cuda()
            p.grad, q.grad = g.clone(), g.clone()
        whole.step()
        pieces.step_groups([2] if it % 2 else [1])
        pieces.step_groups([0, 1] if it % 2 else [0, 2])
    torch.cuda.synchronize()
    for p, q in zip(a, b):
        assert torch.equal(p.detach(), q.detach())
        for k in ("exp_avg", "exp_avg_sq", "kahan_comp"):
            assert torch.equal(whole.state[p][k], pieces.state[q][k])
    assert [int(g["step"]) for g in pieces.param_groups] == [4, 4, 4]
