"""Host-side behaviour that needs no GPU: constructor checks and warnings, state layout, scalar
arithmetic against the reference's formulas, weight-decay groups, low-precision casting, hooks."""

import math
import warnings

import pytest
import torch
from torch import nn

import optimi_b200
from optimi_b200 import _tails as T
from optimi_b200 import functional as F

ALL = [optimi_b200.Adam, optimi_b200.AdamW, optimi_b200.Adan, optimi_b200.Lion, optimi_b200.RAdam, optimi_b200.Ranger,
       optimi_b200.SGD, optimi_b200.StableAdamW]  # fmt: skip


def param(n=16, dtype=torch.float32):
    p = nn.Parameter(torch.zeros(n, dtype=dtype))
    p.grad = torch.ones(n, dtype=dtype)
    return p


@pytest.mark.parametrize("cls", ALL, ids=lambda c: c.__name__)
def test_constructor_validation(cls):
    with pytest.raises(ValueError, match="Invalid learning rate"):
        cls([param()], lr=-1.0)
    with pytest.raises(ValueError, match="Invalid weight decay"):
        cls([param()], lr=1e-3, weight_decay=-0.1)
    if cls is not optimi_b200.SGD:
        with pytest.raises(ValueError, match="Invalid beta1 parameter"):
            cls([param()], lr=1e-3, betas=(1.5, 0.9) if cls is not optimi_b200.Adan else (1.5, 0.9, 0.9))
    else:
        with pytest.raises(ValueError, match="Invalid momentum"):
            cls([param()], lr=1e-3, momentum=1.0)


def test_decouple_lr_defaults_max_lr_and_warns_once_for_high_decay():
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        opt = optimi_b200.AdamW([{"params": [param()], "weight_decay": 1e-2}, {"params": [param()], "weight_decay": 0.1}],
                                lr=2e-3, decouple_lr=True)  # fmt: skip
    assert opt.param_groups[0]["max_lr"] == 2e-3
    msgs = [str(x.message) for x in w if issubclass(x.category, UserWarning)]
    assert len(msgs) == 1 and "up to 0.1" in msgs[0]
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        optimi_b200.AdamW([param()], lr=1e-3, weight_decay=1e-5, decouple_lr=True)
    assert not w


def test_foreach_keyword_is_accepted_with_a_deprecation_warning():
    with pytest.warns(DeprecationWarning):
        optimi_b200.Adam([param()], lr=1e-3, foreach=True)
    optimi_b200.Adam([param()], lr=1e-3, foreach=False, triton=True)  # accepted, ignored


STATE_KEYS = {
    optimi_b200.Adam: {"exp_avg", "exp_avg_sq", "kahan_comp"},
    optimi_b200.AdamW: {"exp_avg", "exp_avg_sq", "kahan_comp"},
    optimi_b200.RAdam: {"exp_avg", "exp_avg_sq", "kahan_comp"},
    optimi_b200.Ranger: {"exp_avg", "exp_avg_sq", "la_param", "kahan_comp"},
    optimi_b200.Lion: {"exp_avg", "kahan_comp"},
    optimi_b200.SGD: {"exp_avg", "kahan_comp"},
    optimi_b200.StableAdamW: {"exp_avg", "exp_avg_sq", "eps_sq", "kahan_comp"},
    optimi_b200.Adan: {"exp_avg", "exp_avg_diff", "exp_avg_sq", "prev_grad", "kahan_comp"},
}


@pytest.mark.parametrize("cls", ALL, ids=lambda c: c.__name__)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_layout_matches_reference(cls, dtype):
    p = param(dtype=dtype)
    p.data.normal_()
    kw = dict(momentum=0.9) if cls is optimi_b200.SGD else {}
    opt = cls([p], lr=1e-3, **kw)
    group, state = opt.param_groups[0], opt.state[p]
    opt._init_state(group, state, p)
    opt._setup_group(group)
    assert set(state) == STATE_KEYS[cls]
    for k, v in state.items():
        if k == "kahan_comp":
            kahan_default_on = dtype == torch.bfloat16 and cls is not optimi_b200.Adan
            assert (v is not None) == kahan_default_on
            if v is not None:
                assert v.dtype == dtype and v.shape == p.shape and not v.any()
        elif k == "eps_sq":
            assert v.ndim == 0 and v.dtype == dtype
        else:
            assert v.dtype == dtype and v.shape == p.shape
    if cls is optimi_b200.Ranger:
        assert torch.equal(state["la_param"], p.data) and state["la_param"].data_ptr() != p.data_ptr()
    if cls is optimi_b200.Adan:
        assert torch.equal(state["prev_grad"], -p.grad)
    assert group["setup"] is True
    has_step = cls not in (optimi_b200.Lion, optimi_b200.SGD)
    assert ("step" in group) == has_step
    if has_step:
        assert group["step"].dtype == torch.int32 and group["step"].device.type == "cpu" and group["step"].ndim == 0


def test_sgd_state_variants():
    p = param()
    opt = optimi_b200.SGD([p], lr=1e-2)
    opt._init_state(opt.param_groups[0], opt.state[p], p)
    assert opt.state[p]["exp_avg"] is None
    p = param()
    p.data.fill_(2.0)
    opt = optimi_b200.SGD([p], lr=1e-2, momentum=0.9, dampening=True, torch_init=True, weight_decay=0.5)
    opt._init_state(opt.param_groups[0], opt.state[p], p)
    assert torch.allclose(opt.state[p]["exp_avg"], torch.full((16,), 2.0))  # g + wd * p = 1 + 0.5 * 2


def test_gradient_release_bookkeeping():
    p = param()
    opt = optimi_b200.Adam([p], lr=1e-3, gradient_release=True)
    assert opt.state[p]["group"] is opt.param_groups[0]
    opt._init_state(opt.param_groups[0], opt.state[p], p)
    assert opt.state[p]["step"].dtype == torch.int32
    assert opt.optimizer_accumulation is False
    opt.optimizer_accumulation = True
    assert opt.optimizer_accumulation is True
    opt.zero_grad(param=p)
    assert p.grad is None


def test_prepare_and_remove_gradient_release():
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    model[1].bias.requires_grad_(False)
    with pytest.raises(ValueError, match="gradient_release=True"):
        optimi_b200.prepare_for_gradient_release(model, optimi_b200.Adam(model.parameters(), lr=1e-3))
    with pytest.raises(TypeError):
        optimi_b200.prepare_for_gradient_release(model, torch.optim.SGD(model.parameters(), lr=1e-3))
    opt = optimi_b200.Adam(model.parameters(), lr=1e-3, gradient_release=True)
    optimi_b200.prepare_for_gradient_release(model, opt)
    assert len(model._gradient_release_hooks) == 3
    with pytest.raises(ValueError, match="already has post_accumulate_grad_hooks"):
        optimi_b200.prepare_for_gradient_release(model, opt)
    optimi_b200.prepare_for_gradient_release(model, opt, ignore_existing_hooks=True)
    optimi_b200.remove_gradient_release(model)
    assert not hasattr(model, "_gradient_release_hooks")
    with pytest.warns(UserWarning):
        optimi_b200.remove_gradient_release(model)


def test_debias_beta_matches_closed_form():
    for beta in (0.9, 0.99, 0.92):
        assert F.debias_beta(beta, 1) == 0
        for t in (2, 5, 100):
            want = beta * (1 - beta ** (t - 1)) / (1 - beta**t)
            assert math.isclose(F.debias_beta(beta, t), want, rel_tol=1e-12)
            assert math.isclose(F.debias(beta, t), 1 - beta**t)


def test_rectification_switches_on_at_step_six_for_beta2_099():
    assert [T.rectification(0.99, t) is not None for t in range(1, 9)] == [False] * 5 + [True] * 3
    rho_inf = 2 / (1 - 0.99) - 1
    assert 0 < T.rectification(0.99, 6) < 1 and abs(T.rectification(0.99, 10**6) - 1) < 1e-3 and rho_inf > 5


def test_param_groups_weight_decay():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(4, 4)
            self.norm = nn.LayerNorm(4)
            self.special = nn.Linear(4, 4, bias=False)
            self.frozen = nn.Linear(4, 4)
            self.frozen.requires_grad_(False)

    net = Net()
    groups = optimi_b200.param_groups_weight_decay(net, 0.1, additional_layers=["special"])
    assert groups[0]["weight_decay"] == 0.0 and groups[1]["weight_decay"] == 0.1
    no_decay = {id(p) for p in groups[0]["params"]}
    assert {id(net.fc.bias), id(net.norm.weight), id(net.norm.bias), id(net.special.weight)} == no_decay
    assert [id(p) for p in groups[1]["params"]] == [id(net.fc.weight)]


def test_to_low_precision_keeps_float32_islands():
    class Rotary(nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("inv_freq", torch.ones(4))

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(10, 4)
            self.fc = nn.Linear(4, 4)
            self.rotary_emb = Rotary()
            self.bn = nn.BatchNorm1d(4)

    net = optimi_b200.to_low_precision(Net())
    assert net.emb.weight.dtype == torch.float32
    assert net.fc.weight.dtype == torch.bfloat16 and net.fc.bias.dtype == torch.bfloat16
    assert net.rotary_emb.inv_freq.dtype == torch.float32
    assert net.bn.running_mean.dtype == torch.bfloat16 and net.bn.num_batches_tracked.dtype == torch.int64
    net = optimi_b200.to_low_precision(Net(), dtype=torch.float16, fp32_modules=None, fp32_buffers=nn.BatchNorm1d)
    assert net.emb.weight.dtype == torch.float16 and net.bn.running_var.dtype == torch.float32 and net.bn.weight.dtype == torch.float16
    with pytest.raises(TypeError):
        optimi_b200.to_low_precision(Net(), fp32_buffers=[3])


def test_empty_step_advances_the_group_counter_like_the_reference():
    p = nn.Parameter(torch.zeros(4))
    opt = optimi_b200.Adam([p], lr=1e-3)
    opt.step()
    assert int(opt.param_groups[0]["step"]) == 1 and opt.param_groups[0]["setup"]


def test_grad_factor_and_graph_entry_points_validate_on_the_host():
    import optimi_b200

    p = torch.nn.Parameter(torch.zeros(8))
    opt = optimi_b200.AdamW([p], lr=1e-3)
    with pytest.raises(ValueError, match="CUDA float32"):
        opt.set_grad_factor(torch.ones(1))  # a CPU tensor
    opt.set_grad_factor(None)
    with pytest.raises(RuntimeError, match="no parameter has a gradient"):
        opt.clip_grad_norm(1.0)
    p.grad = torch.ones(8)
    with pytest.raises(RuntimeError, match="CUDA"):
        opt.clip_grad_norm(1.0)
    with pytest.raises(RuntimeError, match="no captured step"):
        opt.update_graph(None)
    released = optimi_b200.AdamW([p], lr=1e-3, gradient_release=True)
    with pytest.raises(RuntimeError, match="gradient_release"):
        released.clip_grad_norm(1.0)


def test_gradient_layout_must_match_the_parameters():
    """A contiguous gradient for a channels_last (dense but permuted) parameter would be applied to the wrong
    elements: the per-step check refuses it, and accepts a gradient that shares the parameter's strides."""
    from optimi_b200.optimizer import _check_gradient

    p = torch.zeros(2, 3, 4, 5).to(memory_format=torch.channels_last)
    assert not p.is_contiguous()
    with pytest.raises(RuntimeError, match="does not match its parameter"):
        _check_gradient("optimi_b200_adam", torch.zeros(2, 3, 4, 5), p)
    _check_gradient("optimi_b200_adam", torch.zeros_like(p), p)  # zeros_like keeps the layout
    with pytest.raises(RuntimeError, match="does not match its parameter"):
        _check_gradient("optimi_b200_adam", torch.zeros(2, 3, 4, 5, dtype=torch.float64), torch.zeros(2, 3, 4, 5))
    _check_gradient("optimi_b200_adam", torch.zeros(7), torch.zeros(7))


def test_functional_refuses_gradient_release_with_foreach_like_the_reference():
    import optimi_b200.functional as F

    t = torch.zeros(4)
    step = torch.tensor(0, dtype=torch.int32)
    with pytest.raises(ValueError, match="cannot be used together"):
        F.adam(t, t, t, t, lr=1e-3, beta1=0.9, beta2=0.99, weight_decay=0.0, eps=1e-6, step=step, decouple_wd=False,
               foreach=True, gradient_release=True)
    assert int(step) == 1  # the reference advances the counter before it chooses a back end (optimi/adam.py:261-282)
    with pytest.raises(ValueError, match="cannot be used together"):
        F.lion(t, t, t, lr=1e-3, beta1=0.9, beta2=0.99, weight_decay=0.0, foreach=True, gradient_release=True)
