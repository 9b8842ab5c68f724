"""Full-size checks on a B200: properties that do not need an oracle run at that size.

1. Split invariance past 2^31 elements: the step is element-wise, so one 2.1 G-element tensor and the
   same memory cut into a thousand uneven (partly misaligned) views must end bit-identical.  Exercises
   64-bit offsets, the coarse block index, ragged tails and the scalar path at scale.
2. More tensors than one by-value table holds (several launches per step) against the CPU oracle.
3. BASELINE config 2 at full size (1.1 B-parameter Llama-style list, AdamW bf16 + Kahan, decouple_lr,
   50 steps) and the other optimizers of configs 3 and 4 on the same list, against the unmodified
   reference's foreach path on the same GPU, bit for bit (StableAdamW: 1 ulp) — runs only where the
   reference package is present beside the repository (baseline/_ref).
"""

import os
import sys
import warnings

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_free(gb):
    free, _ = torch.cuda.mem_get_info()
    if free < gb * 2**30:
        pytest.skip(f"needs {gb} GiB of free device memory")


def test_split_invariance_beyond_two_to_the_31_elements():
    import optimi_b200.functional as F

    _need_free(60)
    n = (1 << 31) + 4096 + 3
    dt = torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(0)

    def rnd(scale):
        t = torch.empty(n, dtype=dt, device="cuda")
        step = 1 << 27
        for a in range(0, n, step):
            b = min(n, a + step)
            t[a:b] = torch.randn(b - a, device="cuda", generator=gen).mul_(scale).to(dt)
        return t

    base = [rnd(0.02), rnd(1e-3), rnd(1e-3), rnd(1e-6).abs_(), rnd(1e-5)]  # p g m v k
    whole = [t.clone() for t in base]
    parts = [t.clone() for t in base]
    # cut points: some aligned to 8 elements, some not (those pieces take the scalar path)
    cuts = sorted({0, n} | {int(x) for x in torch.randint(1, n - 1, (997,), generator=torch.Generator().manual_seed(1)).tolist()}
                  | {1 << 20, (1 << 30) + 8, (1 << 31) - 1, (1 << 31) + 1})
    views = [[t[a:b] for a, b in zip(cuts[:-1], cuts[1:])] for t in parts]

    kw = dict(lr=3e-4, beta1=0.9, beta2=0.99, weight_decay=1e-5, eps=1e-6, decouple_wd=True, decouple_lr=True, max_lr=3e-4,
              kahan_sum=True)  # fmt: skip
    for s in range(2):
        F.adam([whole[0]], [whole[1]], [whole[2]], [whole[3]], [whole[4]], step=torch.tensor(s, dtype=torch.int32), **kw)
        F.adam(views[0], views[1], views[2], views[3], views[4], step=torch.tensor(s, dtype=torch.int32), **kw)
    torch.cuda.synchronize()
    for name, a, b, ref in zip("pgmvk", whole, parts, base):
        assert torch.equal(a, b), f"{name}: split run differs from whole run"
        if name != "g":
            assert not torch.equal(a[-4096:], ref[-4096:]), f"{name}: tail was not updated"
        else:
            assert torch.equal(a, ref), "gradients must be left untouched"


def test_more_tensors_than_one_table():
    import optimi_b200
    from oracle.port import OracleOptimizer

    gen = torch.Generator().manual_seed(3)
    sizes = [int(x) for x in torch.randint(1, 3000, (1500,), generator=gen)]
    host = [(torch.randn(s, generator=gen) * 0.02).to(torch.bfloat16) for s in sizes]
    grads = [[(torch.randn(s, generator=gen) * 1e-3).to(torch.bfloat16) for s in sizes] for _ in range(3)]
    for name, cls, kw in [("adan", optimi_b200.Adan, dict(lr=3e-4, kahan_sum=True)), ("lion", optimi_b200.Lion, dict(lr=1e-4, weight_decay=0.1))]:
        params = [h.clone().cuda().requires_grad_(True) for h in host]
        opt = cls(params, **kw)
        oracle = OracleOptimizer(name, [h.clone() for h in host], **kw)
        for gs in grads:
            for p, g in zip(params, gs):
                p.grad = g.cuda()
            opt.step()
            oracle.step([g.clone() for g in gs])
        torch.cuda.synchronize()
        bad = [i for i, p in enumerate(params) if not torch.equal(p.detach().cpu(), oracle.params[i])]
        assert not bad, f"{name}: tensors {bad[:10]} differ from the oracle"


REFERENCE_RUNS = [
    # BASELINE config 2: AdamW, decouple_lr, 50 steps
    ("AdamW", dict(lr=3e-4, betas=(0.9, 0.99), weight_decay=1e-5, eps=1e-6, decouple_lr=True), 50, ("exp_avg", "exp_avg_sq", "kahan_comp")),
    # the other optimizers of configs 3 and 4 with their hyper-parameters, on the same 1.1 B list
    ("Lion", dict(lr=1e-4, betas=(0.9, 0.99), weight_decay=0.1), 12, ("exp_avg", "kahan_comp")),
    ("SGD", dict(lr=1e-2, momentum=0.9, weight_decay=1e-2), 12, ("exp_avg", "kahan_comp")),
    ("Adan", dict(lr=3e-4, betas=(0.98, 0.92, 0.99), kahan_sum=True), 30, ("exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp")),
    ("RAdam", dict(lr=3e-4, weight_decay=1e-2, decouple_wd=True), 12, ("exp_avg", "exp_avg_sq", "kahan_comp")),
    ("Ranger", dict(lr=3e-4, k=6, alpha=0.5), 30, ("exp_avg", "exp_avg_sq", "la_param", "kahan_comp")),
    ("StableAdamW", dict(lr=3e-4), 10, ("exp_avg", "exp_avg_sq", "kahan_comp")),
]


@pytest.mark.parametrize("cname,hyper,steps,keys", REFERENCE_RUNS, ids=[r[0] for r in REFERENCE_RUNS])
def test_full_size_against_reference_foreach(cname, hyper, steps, keys):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        pytest.skip("reference package not present beside the repository")
    _need_free(60)
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, ROOT)
    import optimi  # the unmodified reference

    import optimi_b200
    from bench import WORKLOADS, grad_scales, make_params

    shapes = WORKLOADS["llama-1.1b"]()
    mine = [p.requires_grad_(True) for p in make_params(shapes, "cuda", torch.bfloat16, seed=0)]
    theirs = [p.detach().clone().requires_grad_(True) for p in mine]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt_ref = getattr(optimi, cname)(theirs, foreach=True, triton=False, **hyper)
    opt_b200 = getattr(optimi_b200, cname)(mine, **hyper)
    scales = grad_scales(len(shapes), seed=0)
    for step in range(steps):
        gen = torch.Generator(device="cuda").manual_seed(1000 + step)
        for p, q, sc in zip(mine, theirs, scales):
            g = torch.randn(p.shape, device="cuda", generator=gen).mul_(sc).to(torch.bfloat16)
            p.grad = g
            q.grad = g.clone()  # the reference's foreach path clobbers its gradients
        opt_b200.step()
        opt_ref.step()
    torch.cuda.synchronize()
    exact = cname != "StableAdamW"  # its per-tensor mean is summed in another order: 1 bf16 ulp
    for i, (p, q) in enumerate(zip(mine, theirs)):
        pairs = [("param", p.detach(), q.detach())] + [(k, opt_b200.state[p][k], opt_ref.state[q][k]) for k in keys]
        for name, a, b in pairs:
            if exact:
                assert torch.equal(a, b), f"{cname}: {name} of tensor {i} {tuple(p.shape)} differs after {steps} steps"
            else:
                scale = torch.maximum(a.float().abs(), b.float().abs()).clamp_min(1e-3)
                bad = (a.float() - b.float()).abs() > scale * 2.0**-7
                assert not bool(bad.any()), f"{cname}: {name} of tensor {i}: {int(bad.sum())} elements more than 1 ulp apart"


def _compare_with_reference(cname, hyper, steps, keys, shapes, scales, seed_base, label, dtype=torch.bfloat16):
    """Steps `shapes` (one chunk of a parameter list) `steps` times under both implementations with the same
    seeded gradients and compares parameters and states; everything is freed on return."""
    import optimi

    import optimi_b200
    from bench import make_params

    mine = [p.requires_grad_(True) for p in make_params(shapes, "cuda", dtype, seed=seed_base)]
    theirs = [p.detach().clone().requires_grad_(True) for p in mine]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt_ref = getattr(optimi, cname)(theirs, foreach=True, triton=False, **hyper)
    opt_b200 = getattr(optimi_b200, cname)(mine, **hyper)
    for step in range(steps):
        gen = torch.Generator(device="cuda").manual_seed(1000 * seed_base + step)
        for p, q, sc in zip(mine, theirs, scales):
            g = torch.randn(p.shape, device="cuda", generator=gen).mul_(sc).to(dtype)
            p.grad = g
            q.grad = g.clone()  # the reference's foreach path clobbers its gradients
        opt_b200.step()
        opt_ref.step()
    torch.cuda.synchronize()
    exact = cname != "StableAdamW"  # its per-tensor mean is summed in another order: 1 unit of the storage type
    ulp = 2.0**-7 if dtype == torch.bfloat16 else 2.0**-10
    for i, (p, q) in enumerate(zip(mine, theirs)):
        pairs = [("param", p.detach(), q.detach())] + [(k, opt_b200.state[p][k], opt_ref.state[q][k]) for k in keys]
        for name, a, b in pairs:
            if exact:
                assert torch.equal(a, b), f"{cname}, {label}: {name} of tensor {i} {tuple(p.shape)} differs after {steps} steps"
            else:
                scale = torch.maximum(a.float().abs(), b.float().abs()).clamp_min(1e-3)
                bad = (a.float() - b.float()).abs() > scale * ulp
                assert not bool(bad.any()), f"{cname}, {label}: {name} of tensor {i}: {int(bad.sum())} elements more than 1 ulp apart"
    n = sum(p.numel() for p in mine)
    del mine, theirs, opt_ref, opt_b200
    torch.cuda.empty_cache()
    return n


CONFIG3_RUNS = [
    ("AdamW", dict(lr=3e-4, betas=(0.9, 0.99), weight_decay=1e-5, eps=1e-6, decouple_lr=True), ("exp_avg", "exp_avg_sq", "kahan_comp")),
    ("Lion", dict(lr=1e-4, betas=(0.9, 0.99)), ("exp_avg", "kahan_comp")),
    ("SGD", dict(lr=1e-2, momentum=0.9), ("exp_avg", "kahan_comp")),
    ("StableAdamW", dict(lr=3e-4), ("exp_avg", "exp_avg_sq", "kahan_comp")),
]


@pytest.mark.parametrize("cname,hyper,keys", CONFIG3_RUNS, ids=[r[0] for r in CONFIG3_RUNS])
def test_llama3_8b_list_against_reference_foreach_in_chunks(cname, hyper, keys):
    """BASELINE config 3 at its stated size: all 8.03 B parameters of the Llama-3-8B list, bf16 + Kahan, against the
    unmodified reference's foreach path on the same GPU.  Two full copies of the list with their states would not
    fit beside each other, and the step is element-wise, so the list is walked in chunks (the embedding, four
    decoder layers at a time, the head): each chunk is stepped 5 times under both implementations with the same
    seeded gradients, compared bit for bit, and freed."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        pytest.skip("reference package not present beside the repository")
    _need_free(60)
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, ROOT)
    from bench import WORKLOADS, grad_scales

    shapes = WORKLOADS["llama3-8b"]()
    scales = grad_scales(len(shapes), seed=0)
    per_layer = 9
    bounds = [0, 1] + [1 + per_layer * k for k in range(4, 32, 4)] + [1 + per_layer * 32, len(shapes)]
    total = 0
    for c, (a, b) in enumerate(zip(bounds[:-1], bounds[1:])):
        total += _compare_with_reference(cname, hyper, 5, keys, shapes[a:b], scales[a:b], c + 1, f"tensors {a}..{b - 1} of the 8 B list")
    assert total == 8030261248


CONFIG4_RUNS = [
    ("Adan", dict(lr=3e-4, betas=(0.98, 0.92, 0.99), kahan_sum=True), ("exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp")),
    ("Ranger", dict(lr=3e-4, k=6, alpha=0.5), ("exp_avg", "exp_avg_sq", "la_param", "kahan_comp")),
]


@pytest.mark.parametrize("cname,hyper,keys", CONFIG4_RUNS, ids=[r[0] for r in CONFIG4_RUNS])
def test_llama_3b_list_adan_ranger_30_steps_against_reference(cname, hyper, keys):
    """BASELINE config 4 at its stated size and step count: Adan (betas 0.98/0.92/0.99) and Ranger (k=6, alpha=0.5),
    bf16 + Kahan, 30 steps on the whole 3 B Llama-style list at once (both copies with all their state tensors
    resident), bit for bit against the unmodified reference's foreach path on the same GPU."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        pytest.skip("reference package not present beside the repository")
    _need_free(130)
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, ROOT)
    from bench import WORKLOADS, grad_scales

    shapes = WORKLOADS["llama-3b"]()
    scales = grad_scales(len(shapes), seed=0)
    n = _compare_with_reference(cname, hyper, 30, keys, shapes, scales, 7, "the 3 B list")
    assert n == sum(int(torch.Size(s).numel()) for s in shapes)


FP16_RUNS = [
    ("AdamW", dict(lr=3e-4, betas=(0.9, 0.99), weight_decay=1e-5, eps=1e-6, decouple_lr=True), ("exp_avg", "exp_avg_sq", "kahan_comp")),
    ("Adan", dict(lr=3e-4, betas=(0.98, 0.92, 0.99), kahan_sum=True), ("exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp")),
    ("Lion", dict(lr=1e-4, betas=(0.9, 0.99), weight_decay=0.1), ("exp_avg", "kahan_comp")),
]


@pytest.mark.parametrize("cname,hyper,keys", FP16_RUNS, ids=[r[0] for r in FP16_RUNS])
def test_float16_against_reference_foreach(cname, hyper, keys):
    """The float16 kernels (11-bit significands: their own packed Kahan tail, the division shortcut's other operand
    width, the IEEE square root) on the 1.1 B list, 10 steps, bit for bit against the unmodified reference's foreach path."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        pytest.skip("reference package not present beside the repository")
    _need_free(40)
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, ROOT)
    from bench import WORKLOADS, grad_scales

    shapes = WORKLOADS["llama-1.1b"]()
    _compare_with_reference(cname, hyper, 10, keys, shapes, grad_scales(len(shapes), seed=0), 11, "the 1.1 B list in float16", dtype=torch.float16)
