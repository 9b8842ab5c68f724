"""ZeRO-1 style sharding of the optimizer step across the GPUs of one node.

The reference has no distributed code; this is the multi-GPU form of the step the build adds.
Parameters of one dtype are re-pointed into one flat buffer per rank (every rank holds all
parameters, as in data parallelism).  The flat buffer is cut into `world_size` equal element
ranges; a rank keeps optimizer states only for its own range, steps only that range — the step is
element-wise, so a range may start and end in the middle of a tensor — and then one in-place
all-gather over NCCL hands every rank the updated parameters.  Gradients are expected to be already
reduced across ranks (that is the job of the data-parallel layer above the optimizer).

StableAdamW is the one optimizer with a per-tensor quantity (the RMS of g^2/v), so its ranges are
cut on tensor boundaries instead and the exchange is one broadcast per owner of its (unequal) piece.

Exchange modes (`exchange=`):
    "nccl"   step the local range, then all-gather (works everywhere, any optimizer).
    "push"   the flat buffers are symmetric-memory allocations mapped into every rank; the step kernel
             itself stores each updated parameter vector into every peer's buffer over NVLink as it
             goes (`optimi_b200_push_begin` around the step), so the exchange overlaps the step tile
             by tile.  The ranks then meet in a one-element all-reduce on the same stream, which
             orders every rank's later work after all pushes.  Needs an optimi_b200 optimizer on 2-8
             CUDA ranks and one parameter dtype; anything else falls back to "nccl".
    "auto"   "push" when available, else "nccl".

`reduce_grads=True` (with the push exchange) also folds the data-parallel gradient reduction into the
step: gradients live in a second symmetric flat buffer (`attach_grads()` points every `p.grad` into it,
so autograd accumulates there), and the step kernel reads, for each element of its range, the gradient
of every rank over NVLink, averages them in fp32 in rank order and rounds once — reduce-scatter, step
and all-gather in one launch, with one tiny collective before it (all gradients written) and one
after it (all reads and pushes done).  Not available for StableAdamW.

Sharded and unsharded runs produce bit-identical parameters: each element sees exactly the same
arithmetic, only on another GPU.
"""

from __future__ import annotations

import os
from typing import Any, Callable

import torch
import torch.distributed as dist
from torch import Tensor

ALIGN_ELEMS = 256  # shard and tensor starts are multiples of this many elements (>= 16 bytes for every dtype)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatLayout:
    """Where each tensor of one dtype group sits in the flat buffer, and which slice each rank owns."""

    def __init__(self, numels: list[int], world_size: int, split_on_tensors: bool = False):
        self.numels = list(numels)
        self.offsets = []
        off = 0
        for n in numels:
            self.offsets.append(off)
            off = _round_up(off + n, ALIGN_ELEMS)
        self.total = _round_up(off, ALIGN_ELEMS * world_size)
        self.world_size = world_size
        if not split_on_tensors:
            per = self.total // world_size
            self.bounds = [r * per for r in range(world_size + 1)]
        else:
            # boundaries on tensor starts, each as close as possible to the equal split
            starts = self.offsets + [self.total]
            self.bounds = [0]
            for r in range(1, world_size):
                target = r * self.total / world_size
                best = min(starts, key=lambda s: abs(s - target))
                self.bounds.append(max(best, self.bounds[-1]))
            self.bounds.append(self.total)

    def rank_range(self, rank: int) -> tuple[int, int]:
        return self.bounds[rank], self.bounds[rank + 1]

    def pieces(self, rank: int) -> list[tuple[int, int, int]]:
        """(tensor index, start element within the tensor, end element) of every tensor part in `rank`'s range."""
        lo, hi = self.rank_range(rank)
        out = []
        for i, (off, n) in enumerate(zip(self.offsets, self.numels)):
            a, b = max(lo, off), min(hi, off + n)
            if a < b:
                out.append((i, a - off, b - off))
        return out


class ShardedOptimizer:
    """Wraps one optimi_b200 (or any torch) optimizer class so that each rank steps 1/world of the elements.

    Args:
        optimizer_cls: the optimizer class, e.g. ``optimi_b200.AdamW``.
        params: parameters (one group).  Their storage is moved into flat buffers, values preserved.
        process_group: the ranks to shard over (default: the world group).
        split_on_tensors: cut ranges on tensor boundaries (set automatically for StableAdamW).
        gather: ``"nccl"`` (all-gather after the step) or a callable ``gather(flat, lo, hi)``.
        **kwargs: passed to the optimizer constructor.
    """

    def __init__(self, optimizer_cls: Callable, params, process_group=None, split_on_tensors: bool | None = None,
                 gather: str | Callable = "nccl", exchange: str = "nccl", reduce_grads: bool = False, **kwargs: Any):  # fmt: skip
        self.group = process_group
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.params = [p for p in params]
        if split_on_tensors is None:
            split_on_tensors = getattr(optimizer_cls, "__name__", "") == "StableAdamW"
        self.gather = gather
        can_push = (
            self.world > 1 and self.world <= 8 and hasattr(optimizer_cls, "_c_fn")
            and all(p.is_cuda for p in self.params) and len({(p.device, p.dtype) for p in self.params}) == 1
        )  # fmt: skip
        if exchange == "push" and not can_push:
            raise ValueError("exchange='push' needs 2-8 CUDA ranks, one parameter dtype and an optimi_b200 optimizer")
        self.exchange = "push" if (exchange in ("push", "auto") and can_push) else "nccl"
        self._peer_deltas: list[int] | None = None
        self._symm_handles = []
        if reduce_grads and (self.exchange != "push" or split_on_tensors):
            raise ValueError("reduce_grads=True needs the push exchange and an optimizer other than StableAdamW")
        self.reduce_grads = reduce_grads
        self._grad_deltas: list[int] | None = None

        # one flat buffer per (device, dtype)
        self.buckets: list[dict[str, Any]] = []
        groups: dict[tuple, list[Tensor]] = {}
        for p in self.params:
            groups.setdefault((p.device, p.dtype), []).append(p)
        shard_params: list[Tensor] = []
        for (device, dtype), plist in groups.items():
            layout = FlatLayout([p.numel() for p in plist], self.world, split_on_tensors)
            grad_flat = grad_handle = None
            if self.exchange == "push":
                flat, _, self._peer_deltas = self._symmetric_buffer(layout.total, dtype, device)
                if reduce_grads:
                    grad_flat, grad_handle, others = self._symmetric_buffer(layout.total, dtype, device)
                    others = iter(others)  # all ranks in rank order, 0 for this one
                    self._grad_deltas = [0 if r == self.rank else next(others) for r in range(self.world)]
            else:
                flat = torch.zeros(layout.total, dtype=dtype, device=device)
            for p, off in zip(plist, layout.offsets):
                view = flat[off : off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
            pieces = layout.pieces(self.rank)
            shards = []
            for i, a, b in pieces:
                sp = torch.nn.Parameter(plist[i].data.view(-1)[a:b], requires_grad=True)
                shards.append(sp)
            shard_params.extend(shards)
            self.buckets.append(dict(layout=layout, flat=flat, params=plist, pieces=pieces, shards=shards, grad_flat=grad_flat,
                                     grad_handle=grad_handle))
        self.shard_params = shard_params
        self.inner = optimizer_cls(shard_params, **kwargs)
        if self.exchange == "push":
            self._meet = torch.zeros(1, dtype=torch.int32, device=self.params[0].device)
            # no rank may start pushing before every rank has finished filling its own buffer
            torch.cuda.synchronize(self.params[0].device)
            dist.barrier(self.group)

    def _symmetric_buffer(self, numel: int, dtype: torch.dtype, device: torch.device):
        """A zeroed buffer every rank of the group can load from and store into: torch symmetric memory
        (CUDA virtual memory handles exchanged between the ranks); only plain peer loads and stores are
        used on it.  Returns (buffer, handle, byte offsets from this rank's buffer to each peer's)."""
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        flat = symm.empty(numel, dtype=dtype, device=device)
        handle = symm.rendezvous(flat, self.group if self.group is not None else dist.group.WORLD)
        flat.zero_()
        base = flat.data_ptr()
        ptrs = list(handle.buffer_ptrs)
        if ptrs[self.rank] != base:
            raise RuntimeError("symmetric memory: this rank's buffer pointer does not match the allocation")
        deltas = [ptrs[r] - base for r in range(self.world) if r != self.rank]
        self._symm_handles.append(handle)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)
        return flat, handle, deltas

    # convenience passthroughs ------------------------------------------------------------------
    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def state(self):
        return self.inner.state

    def local_elements(self) -> int:
        return sum(sp.numel() for sp in self.shard_params)

    def attach_grads(self) -> None:
        """reduce_grads only: points every parameter's `.grad` at its (zeroed) slot of the shared gradient
        buffer, so that the backward pass accumulates where the other ranks' step kernels can read."""
        for b in self.buckets:
            gf, layout = b["grad_flat"], b["layout"]
            for p, off in zip(b["params"], layout.offsets):
                p.grad = gf[off : off + p.numel()].view(p.shape)

    def _bind_grads(self):
        if self.reduce_grads:
            for b in self.buckets:
                gf, layout = b["grad_flat"], b["layout"]
                for (i, a, e), sp in zip(b["pieces"], b["shards"]):
                    g = b["params"][i].grad
                    off = layout.offsets[i]
                    if g is None or g.data_ptr() != gf.data_ptr() + off * gf.element_size():
                        raise RuntimeError("reduce_grads=True: call attach_grads() before the backward pass (gradients must live in the shared buffer)")
                    sp.grad = gf[off + a : off + e]
            return
        for b in self.buckets:
            for (i, a, e), sp in zip(b["pieces"], b["shards"]):
                g = b["params"][i].grad
                if g is None:
                    sp.grad = None
                    continue
                if not g.is_contiguous():
                    raise RuntimeError("ShardedOptimizer needs contiguous gradients")
                sp.grad = g.view(-1)[a:e]

    @torch.no_grad()
    def step_local(self, shard_grads: list[Tensor] | None = None):
        """Steps this rank's range only (no exchange).  `shard_grads`, one tensor per entry of
        `shard_params`, bypasses the parameters' `.grad` (a rank that received only its slice of the
        gradients from a reduce-scatter has nothing else)."""
        if shard_grads is None:
            self._bind_grads()
        else:
            for sp, g in zip(self.shard_params, shard_grads):
                sp.grad = g
        if self.exchange == "push":
            from ._lib import peer_pull, peer_push

            if self.reduce_grads:
                if shard_grads is not None:
                    raise ValueError("reduce_grads=True reads the gradients of the shared buffer; do not pass shard_grads")
                dist.all_reduce(self._meet, group=self.group)  # every rank's gradients are written
                self._init_states_from_mean_gradients()
                with peer_pull(self._grad_deltas, 1.0 / self.world), peer_push(self._peer_deltas):
                    self.inner.step()
            else:
                with peer_push(self._peer_deltas):
                    self.inner.step()
        else:
            self.inner.step()

    def _init_states_from_mean_gradients(self) -> None:
        """reduce_grads, first step only.  Some optimizers seed their state from the first gradient
        (Adan's previous gradient, SGD's `torch_init` momentum); the fused step never materialises the
        averaged gradient, so it is computed here once, with the kernel's own arithmetic (fp32 sum in
        rank order, times 1/world, one rounding), just for the state constructors."""
        if getattr(self, "_states_seeded", False) or not hasattr(self.inner, "_init_state"):
            return
        self._states_seeded = True
        torch.cuda.current_stream().synchronize()  # the meeting collective above has completed: all gradients are in place
        group = self.inner.param_groups[0]
        for b in self.buckets:
            layout, gf, handle = b["layout"], b["grad_flat"], b["grad_handle"]
            views = [handle.get_buffer(r, (layout.total,), gf.dtype) if r != self.rank else gf for r in range(self.world)]
            for (i, a, e), sp in zip(b["pieces"], b["shards"]):
                lo = layout.offsets[i] + a
                acc = views[0][lo : lo + e - a].float()
                for v in views[1:]:
                    acc = acc + v[lo : lo + e - a].float()
                bound = sp.grad
                sp.grad = (acc * (1.0 / self.world)).to(gf.dtype)
                self.inner._init_state(group, self.inner.state[sp], sp)
                sp.grad = bound
        torch.cuda.synchronize()
        dist.barrier(self.group)

    @torch.no_grad()
    def gather_params(self):
        """Hands every rank the updated parameters: one in-place all-gather per flat buffer."""
        if self.world == 1:
            return
        if self.exchange == "push":
            # the step kernel already stored this rank's range into every peer; meeting in a tiny
            # collective on the stream orders all later work after every rank's pushes
            dist.all_reduce(self._meet, group=self.group)
            return
        for b in self.buckets:
            layout, flat = b["layout"], b["flat"]
            lo, hi = layout.rank_range(self.rank)
            if callable(self.gather):
                self.gather(flat, lo, hi)
                continue
            sizes = [layout.bounds[r + 1] - layout.bounds[r] for r in range(self.world)]
            if all(s == sizes[0] for s in sizes):
                dist.all_gather_into_tensor(flat, flat[lo:hi], group=self.group)
            else:
                # unequal pieces (ranges cut on tensor boundaries): one broadcast per owner
                for r in range(self.world):
                    piece = flat[layout.bounds[r] : layout.bounds[r + 1]]
                    if piece.numel():
                        src = dist.get_global_rank(self.group, r) if self.group is not None else r
                        dist.broadcast(piece, src=src, group=self.group)

    @torch.no_grad()
    def step(self, shard_grads: list[Tensor] | None = None):
        if torch.cuda.is_initialized() and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("ShardedOptimizer.step() cannot be captured into a CUDA graph")
        self.step_local(shard_grads)
        self.gather_params()

    def zero_grad(self, set_to_none: bool = True):
        if self.reduce_grads:  # gradients stay attached to the shared buffer; call after step() (its closing collective
            for b in self.buckets:  # guarantees no rank is still reading)
                b["grad_flat"].zero_()
            return
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()
        for sp in self.shard_params:
            sp.grad = None

    # checkpoints -------------------------------------------------------------------------------
    def _exchange(self, flat: Tensor, layout: FlatLayout) -> None:
        """Every rank ends up with all ranks' ranges of `flat` (each rank has filled its own)."""
        if self.world == 1:
            return
        lo, hi = layout.rank_range(self.rank)
        sizes = {layout.bounds[r + 1] - layout.bounds[r] for r in range(self.world)}
        if len(sizes) == 1:
            dist.all_gather_into_tensor(flat, flat[lo:hi].clone(), group=self.group)
        else:
            for r in range(self.world):
                piece = flat[layout.bounds[r] : layout.bounds[r + 1]]
                if piece.numel():
                    src = dist.get_global_rank(self.group, r) if self.group is not None else r
                    dist.broadcast(piece, src=src, group=self.group)

    def consolidated_state_dict(self) -> dict[str, Any]:
        """The optimizer state in the UNSHARDED layout of the wrapped optimizer class — what
        `optimizer_cls(params).state_dict()` would hold after the same steps — on every rank.  Per-element
        state tensors are put back together from the ranks' ranges; everything else (step counters,
        0-dim tensors, None) is taken from the rank that owns the tensor's first element.  A collective:
        all ranks must call it.  The result loads into a plain optimizer of the reference or of this
        package, or into a `ShardedOptimizer` of any world size (`load_consolidated_state_dict`)."""
        index_of = {id(p): i for i, p in enumerate(self.params)}
        state: dict[int, dict[str, Any]] = {}
        for b in self.buckets:
            layout, plist = b["layout"], b["params"]
            device, dtype = b["flat"].device, b["flat"].dtype
            local = {}
            for (i, a, e), sp in zip(b["pieces"], b["shards"]):
                local[(i, a, e)] = self.inner.state.get(sp, {})
            elem_keys, other = set(), {}
            for (i, a, e), st in local.items():
                for k, v in st.items():
                    if torch.is_tensor(v) and v.dim() > 0 and v.numel() == e - a:
                        elem_keys.add(k)
                    elif a == 0:
                        other.setdefault(i, {})[k] = v.cpu() if torch.is_tensor(v) else v
            if self.world > 1:
                gathered = [None] * self.world
                dist.all_gather_object(gathered, (sorted(elem_keys), other), group=self.group)
                elem_keys = set().union(*[set(g[0]) for g in gathered])
                other = {i: kv for g in gathered for i, kv in g[1].items()}
            for i, p in enumerate(plist):
                state[index_of[id(p)]] = dict(other.get(i, {}))
            for k in sorted(elem_keys):
                flat = torch.zeros(layout.total, dtype=dtype, device=device)
                for (i, a, e), st in local.items():
                    if st.get(k) is not None:
                        flat[layout.offsets[i] + a : layout.offsets[i] + e] = st[k].reshape(-1)
                self._exchange(flat, layout)
                for i, p in enumerate(plist):
                    off = layout.offsets[i]
                    state[index_of[id(p)]][k] = flat[off : off + p.numel()].view(p.shape).clone()
                del flat
        groups = []
        for g in self.inner.param_groups:
            groups.append({k: v for k, v in g.items() if k != "params"} | {"params": list(range(len(self.params)))})
        # parameters that never received a gradient have no state, as in an unsharded optimizer
        state = {i: st for i, st in state.items() if st}
        return {"state": state, "param_groups": groups}

    def load_consolidated_state_dict(self, sd: dict[str, Any]) -> None:
        """Loads an unsharded state dict (from `consolidated_state_dict`, from a plain optimizer of this
        package or from the reference): every rank keeps the slices of its own range."""
        inner_sd = self.inner.state_dict()
        order = [sp for b in self.buckets for sp in b["shards"]]
        piece_of = [(b, piece) for b in self.buckets for piece in b["pieces"]]
        index_of = {id(p): i for i, p in enumerate(self.params)}
        new_state = {}
        for j, (sp, (b, (i, a, e))) in enumerate(zip(order, piece_of)):
            full = sd["state"].get(index_of[id(b["params"][i])])
            if full is None:
                continue
            entry = {}
            for k, v in full.items():
                if torch.is_tensor(v) and v.dim() > 0 and v.numel() == b["params"][i].numel():
                    entry[k] = v.reshape(-1)[a:e].clone()
                else:
                    entry[k] = v.clone() if torch.is_tensor(v) else v
            new_state[j] = entry
        groups = []
        for g_new, g_old in zip(sd["param_groups"], inner_sd["param_groups"]):
            groups.append({k: v for k, v in g_new.items() if k != "params"} | {"params": g_old["params"]})
        self.inner.load_state_dict({"state": new_state, "param_groups": groups})

    def state_dict(self) -> dict[str, Any]:
        """This rank's shard of the optimizer state plus the layout needed to put shards back together."""
        return {
            "inner": self.inner.state_dict(),
            "rank": self.rank,
            "world": self.world,
            "pieces": [b["pieces"] for b in self.buckets],
        }

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if sd["world"] != self.world or sd["rank"] != self.rank:
            raise ValueError(f"shard of rank {sd['rank']}/{sd['world']} loaded into rank {self.rank}/{self.world}")
        self.inner.load_state_dict(sd["inner"])
