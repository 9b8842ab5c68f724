"""The reference's canonical model preparation, stepped by both implementations on the same GPU.

optimi's users cast a model with `to_low_precision` (float32 embeddings beside a bfloat16 body,
optimi/utils.py:104-169, tested by the reference in tests/test_to_low_precision.py:47-109) and split
it with `param_groups_weight_decay` (biases and norm weights without decay, optimi/utils.py:41-71,
tests/test_weight_decay.py:30-125): two parameter groups x two dtypes in one optimizer.  Here a
GPT-shaped toy prepared that way trains for 20 steps (real forward and backward passes) under
`optimi_b200` and, with the very same gradients, under the unmodified reference's foreach path;
parameters and every state tensor must agree bit for bit, the float32 embedding included.

Needs the reference package beside the repository (baseline/_ref), which travels with it.
"""

import os
import sys
import warnings

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "optimi")):
        pytest.skip("reference package not present beside the repository")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    import optimi

    return optimi


class Block(nn.Module):
    def __init__(self, d, f):
        super().__init__()
        self.norm, self.up, self.down = nn.LayerNorm(d), nn.Linear(d, f), nn.Linear(f, d)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm(x))))


class ToyGPT(nn.Module):
    def __init__(self, vocab=1000, d=128, f=512, layers=2):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList([Block(d, f) for _ in range(layers)])
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, idx):
        x = self.embed(idx).to(self.head.weight.dtype)
        for b in self.blocks:
            x = b(x)
        return self.head(self.norm(x))


CASES = [
    ("AdamW", dict(lr=1e-3, betas=(0.9, 0.99), eps=1e-6), ("exp_avg", "exp_avg_sq", "kahan_comp"), True),
    ("Adam", dict(lr=1e-3, weight_decay=1e-2), ("exp_avg", "exp_avg_sq", "kahan_comp"), True),  # L2 decay
    ("Lion", dict(lr=1e-4, betas=(0.9, 0.99)), ("exp_avg", "kahan_comp"), True),
    ("SGD", dict(lr=1e-2, momentum=0.9), ("exp_avg", "kahan_comp"), True),
    ("Adan", dict(lr=1e-3, kahan_sum=True), ("exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp"), True),
    ("Ranger", dict(lr=1e-3, k=3), ("exp_avg", "exp_avg_sq", "la_param", "kahan_comp"), True),
    ("StableAdamW", dict(lr=1e-3), ("exp_avg", "exp_avg_sq", "kahan_comp"), False),
]


@pytest.mark.parametrize("cname,kw,keys,exact", CASES, ids=[c[0] for c in CASES])
def test_low_precision_model_with_weight_decay_groups(cname, kw, keys, exact):
    optimi = _reference()
    import optimi_b200

    dev = torch.device("cuda")
    torch.manual_seed(0)
    mine = optimi_b200.to_low_precision(ToyGPT(), device=dev)
    theirs = optimi.to_low_precision(ToyGPT(), device=dev)
    theirs.load_state_dict(mine.state_dict())
    assert mine.embed.weight.dtype == torch.float32 and mine.head.weight.dtype == torch.bfloat16
    assert [p.dtype for p in mine.parameters()] == [p.dtype for p in theirs.parameters()]

    groups_mine = optimi_b200.param_groups_weight_decay(mine, weight_decay=1e-2)
    groups_theirs = optimi.param_groups_weight_decay(theirs, weight_decay=1e-2)
    assert [[tuple(p.shape) for p in g["params"]] for g in groups_mine] == [[tuple(p.shape) for p in g["params"]] for g in groups_theirs]
    assert [g["weight_decay"] for g in groups_mine] == [g["weight_decay"] for g in groups_theirs]
    if "weight_decay" in kw:  # one decay for every group, passed as the optimizer's default
        groups_mine, groups_theirs = list(mine.parameters()), list(theirs.parameters())
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt_mine = getattr(optimi_b200, cname)(groups_mine, **kw)
        opt_theirs = getattr(optimi, cname)(groups_theirs, foreach=True, triton=False, **kw)

    gen = torch.Generator(device=dev).manual_seed(1)
    for _ in range(20):
        idx = torch.randint(0, 1000, (8, 64), device=dev, generator=gen)
        loss = torch.nn.functional.cross_entropy(mine(idx).float().view(-1, 1000), idx.view(-1))
        loss.backward()
        for p, q in zip(mine.parameters(), theirs.parameters()):
            q.grad = p.grad.clone()  # the same gradients for both; the reference's foreach path uses its copy as scratch
        opt_mine.step()
        opt_theirs.step()
        opt_mine.zero_grad()
        opt_theirs.zero_grad()
    torch.cuda.synchronize()

    for (name, p), q in zip(mine.named_parameters(), theirs.parameters()):
        pairs = [("param", p.detach(), q.detach())]
        for k in keys:
            a, b = opt_mine.state[p].get(k), opt_theirs.state[q].get(k)
            assert (a is None) == (b is None), f"{name}: state `{k}` exists in one implementation only"
            if a is not None:
                pairs.append((k, a, b))
        for what, a, b in pairs:
            assert a.dtype == b.dtype, f"{name}: {what} is {a.dtype} here and {b.dtype} in the reference"
            if exact:
                assert torch.equal(a, b), f"{cname}: {what} of {name} ({a.dtype}) differs from the reference after 20 steps"
            else:  # StableAdamW sums its per-tensor mean in another order: 1e-6 relative (float32) / 1 ulp (bfloat16)
                tol = 1e-6 if a.dtype == torch.float32 else 2.0**-7
                scale = torch.maximum(a.float().abs(), b.float().abs()).clamp_min(1e-3)
                bad = (a.float() - b.float()).abs() > scale * tol
                assert not bool(bad.any()), f"{cname}: {what} of {name} ({a.dtype}): {int(bad.sum())} elements beyond tolerance"
