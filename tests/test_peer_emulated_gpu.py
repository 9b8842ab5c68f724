"""The fused "reduce-scatter + step + all-gather" kernels for up to eight ranks, exercised on ONE GPU.

The step kernels never wait on another rank: a launch reads the gradient of every rank through byte
offsets from its own gradient buffer, adds them in rank order, steps its own range and stores the
updated parameters at byte offsets from its own parameter buffer.  Nothing requires the other
buffers to live on other GPUs.  So the ranks of a sharded run can be played one after another on one
device — every "rank" gets its own copy of the parameters and its own full gradients, all in this
GPU's memory — and the outcome must be what an unsharded optimizer makes of the mean gradient, in
every rank's copy.  This runs the rank-bound-2, -4 and -8 kernels (and rank counts below a bound)
without needing that many GPUs; the real multi-GPU runs are in tests/test_zero_gpu.py.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mean_gradient(grads, world):
    acc = grads[0].float()
    for g in grads[1:]:
        acc = acc + g.float()
    return (acc * (1.0 / world)).to(grads[0].dtype)  # fp32 sum in rank order, times 1/world, one rounding


@pytest.mark.parametrize("per_rank", [4096 * 3 + 8, 5001], ids=["aligned-ranges", "misaligned-ranges"])
@pytest.mark.parametrize("world", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("which", ["adamw", "lion", "adan"])
def test_all_ranks_played_on_one_gpu_equal_unsharded_step_on_mean_gradient(which, world, per_rank):
    import optimi_b200
    import optimi_b200.functional as F
    from optimi_b200._lib import peer_pull, peer_push

    total = per_rank * world
    total_padded = (total + 7) // 8 * 8  # rows 16 bytes apart in whole vectors
    dev, dt = torch.device("cuda"), torch.bfloat16
    gen = torch.Generator().manual_seed(world * 100 + per_rank % 97)
    init = (torch.randn(total, generator=gen) * 0.02).to(dt)
    params = torch.zeros(world, total_padded, dtype=dt, device=dev)  # one copy of all parameters per rank
    params[:, :total] = init.to(dev)
    grads = torch.zeros(world, total_padded, dtype=dt, device=dev)  # every rank's own full gradients
    row_bytes = total_padded * 2

    def states(n):
        return [torch.zeros(per_rank, dtype=dt, device=dev) for _ in range(n)]

    n_states = {"adamw": 3, "lion": 2, "adan": 5}[which]  # per rank: its range only
    rank_states = [states(n_states) for _ in range(world)]
    steps = [torch.tensor(0, dtype=torch.int32) for _ in range(world)]

    twin = torch.nn.Parameter(init.clone().to(dev))
    if which == "adamw":
        kw = dict(lr=3e-4, weight_decay=1e-2)
        plain = optimi_b200.AdamW([twin], **kw)
    elif which == "lion":
        kw = dict(lr=1e-4, weight_decay=0.1)
        plain = optimi_b200.Lion([twin], **kw)
    else:
        kw = dict(lr=3e-4, kahan_sum=True)
        plain = optimi_b200.Adan([twin], **kw)

    for it in range(3):
        for r in range(world):
            grads[r, :total] = (torch.randn(total, generator=gen) * 1e-3).to(dt).to(dev)
        mean = _mean_gradient([grads[r, :total] for r in range(world)], world)
        if which == "adan" and it == 0:
            # Adan's previous-gradient state starts as the negated first (mean) gradient, as the sharded wrapper seeds it
            for r in range(world):
                rank_states[r][3].copy_(-mean[r * per_rank : (r + 1) * per_rank])
        for r in range(world):
            lo, hi = r * per_rank, (r + 1) * per_rank
            p, g = params[r, lo:hi], grads[r, lo:hi]
            pull = [(s - r) * row_bytes for s in range(world)]  # to every rank's gradients, 0 for this one
            push = [(s - r) * row_bytes for s in range(world) if s != r]  # to every other rank's parameters
            st = rank_states[r]
            with torch.no_grad(), peer_pull(pull, 1.0 / world), peer_push(push):
                if which == "adamw":
                    F.adamw([p], [g], [st[0]], [st[1]], [st[2]], lr=3e-4, beta1=0.9, beta2=0.99, weight_decay=1e-2, eps=1e-6,
                            step=steps[r], kahan_sum=True)
                elif which == "lion":
                    F.lion([p], [g], [st[0]], [st[1]], lr=1e-4, beta1=0.9, beta2=0.99, weight_decay=0.1, kahan_sum=True)
                else:
                    F.adan([p], [g], [st[0]], [st[1]], [st[2]], [st[3]], [st[4]], lr=3e-4, beta1=0.98, beta2=0.92, beta3=0.99,
                           weight_decay=2e-2, eps=1e-6, step=steps[r], kahan_sum=True)
        twin.grad = mean
        plain.step()
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(params[r, :total], twin.detach()), f"rank {r}'s copy differs from the unsharded step on the mean gradient"
    assert bool((grads[:, total:] == 0).all()) and bool((params[:, total:] == 0).all()), "something was written past the lists"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_push_only_with_all_ranks_on_one_gpu(world):
    """The plain sharded step (gradients already reduced, the step kernel only pushes its updated range to up to
    seven peers): after all ranks have been played, every copy equals the unsharded step."""
    import optimi_b200
    import optimi_b200.functional as F
    from optimi_b200._lib import peer_push

    per_rank = 4096 * 2 + 264
    total = per_rank * world
    dev, dt = torch.device("cuda"), torch.bfloat16
    gen = torch.Generator().manual_seed(world)
    init = (torch.randn(total, generator=gen) * 0.02).to(dt)
    params = init.to(dev).repeat(world, 1).contiguous()
    row_bytes = total * 2
    st = [[torch.zeros(per_rank, dtype=dt, device=dev) for _ in range(3)] for _ in range(world)]
    steps = [torch.tensor(0, dtype=torch.int32) for _ in range(world)]
    twin = torch.nn.Parameter(init.clone().to(dev))
    plain = optimi_b200.AdamW([twin], lr=3e-4, weight_decay=1e-2)
    for _ in range(3):
        grad = (torch.randn(total, generator=gen) * 1e-3).to(dt).to(dev)
        for r in range(world):
            lo, hi = r * per_rank, (r + 1) * per_rank
            with torch.no_grad(), peer_push([(s - r) * row_bytes for s in range(world) if s != r]):
                F.adamw([params[r, lo:hi]], [grad[lo:hi]], [st[r][0]], [st[r][1]], [st[r][2]], lr=3e-4, beta1=0.9, beta2=0.99,
                        weight_decay=1e-2, eps=1e-6, step=steps[r], kahan_sum=True)
        twin.grad = grad
        plain.step()
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(params[r], twin.detach()), f"rank {r}'s copy differs from the unsharded step"
