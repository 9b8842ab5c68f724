"""ZeRO-1 style sharding of the optimizer step across the GPUs of one node.

The reference has no distributed code; this is the multi-GPU form of the step the build adds.
Parameters are re-pointed into one flat buffer per dtype on every rank (every rank holds all
parameters, as in data parallelism).  Each flat buffer is cut into `world_size` equal element
ranges; a rank keeps optimizer states only for its own range, steps only that range — the step is
element-wise, so a range may start and end in the middle of a tensor — and then the updated
parameters reach the other ranks.  Gradients are expected to be already reduced across ranks (that
is the job of the data-parallel layer above the optimizer) unless `reduce_grads=True`.

`params` may be a list of tensors or a list of param-group dicts with per-group options, as for any
torch optimizer (`param_groups_weight_decay(model)` returns two groups); parameters of several
dtypes (`to_low_precision(model)` keeps embeddings in float32) get one flat buffer each.

StableAdamW is the one optimizer with a per-tensor quantity (the RMS of g^2/v), so its ranges are
cut on tensor boundaries instead and the exchange is one broadcast per owner of its (unequal) piece.

Exchange modes (`exchange=`):
    "nccl"   step the local range, then all-gather (works everywhere, any optimizer).
    "push"   the flat buffers live in one symmetric-memory allocation mapped into every rank; the step
             kernel itself stores each updated parameter vector into every peer's buffer over NVLink
             as it goes (`optimi_b200_push_begin` around the step), so the exchange overlaps the step
             tile by tile.  Needs an optimi_b200 optimizer on 2-8 CUDA ranks; anything else falls
             back to "nccl".
    "auto"   "push" when available, else "nccl".

Ordering under "push".  A rank's step stores into its peers' LIVE parameter buffers, so two things
must hold.  Before: no peer may still be reading the parameters (its forward, backward or an
evaluation pass) when this rank starts to push; `pre_step_sync=True` (the default) makes the ranks
meet in a one-element all-reduce on the current stream right before the step, which orders every
rank's earlier work on that stream ahead of every rank's pushes.  Switch it off only when a
blocking collective on the same stream (the gradient all-reduce or reduce-scatter of the
data-parallel layer) already separates the last use of the parameters from `step()`.  After: the
ranks meet again in the same way after the launch, so that whatever a rank enqueues next sees all
ranks' pushes.

`reduce_grads=True` (with the push exchange) also folds the data-parallel gradient reduction into the
step: gradients live in a second symmetric allocation (`attach_grads()` points every `p.grad` into it,
so autograd accumulates there), and the step kernel reads, for each element of its range, the gradient
of every rank over NVLink, averages them in fp32 in rank order and rounds once — reduce-scatter, step
and all-gather in one launch, with one tiny collective before it (all gradients written) and one
after it (all reads and pushes done).  Not available for StableAdamW.

Sharded and unsharded runs produce bit-identical parameters: each element sees exactly the same
arithmetic, only on another GPU.  `check_replicas()` verifies on demand that all ranks hold the same
bits.

Host-side failure detection: the constructor makes the ranks compare a digest of what they were
given (group structure, sizes, dtypes, options that shape the layout) BEFORE anything is allocated
or launched, and raises on every rank when they differ — with the push exchange a rank whose list
differed would otherwise store through peer mappings at offsets its peers never laid out.
"""

from __future__ import annotations

import hashlib
import os
from typing import Any, Callable

import torch
import torch.distributed as dist
from torch import Tensor

ALIGN_ELEMS = 256  # shard and tensor starts are multiples of this many elements (>= 16 bytes for every dtype)
ARENA_ALIGN = 4096  # byte alignment of each dtype's region inside a symmetric allocation
CHECKSUM_CHUNK = 1 << 26  # elements per partial checksum of `replica_checksums`


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


def _as_groups(params) -> list[dict[str, Any]]:
    """`params` as a list of param-group dicts (torch.optim.Optimizer accepts tensors or dicts)."""
    params = list(params)
    if not params:
        raise ValueError("ShardedOptimizer got an empty parameter list")
    if isinstance(params[0], dict):
        groups = []
        for g in params:
            ps = g["params"]
            groups.append({**g, "params": [ps] if isinstance(ps, Tensor) else list(ps)})
        return groups
    return [{"params": params}]


def layout_digest(groups: list[dict[str, Any]], world: int, *extra: Any) -> str:
    """A digest of everything that decides where each rank puts what: the group structure, every
    parameter's size and dtype, the world size and `extra` (optimizer class, split and exchange mode)."""
    desc = (world, extra, [[(p.numel(), str(p.dtype)) for p in g["params"]] for g in groups])
    return hashlib.sha256(repr(desc).encode()).hexdigest()


def assert_ranks_agree(digest: str, group=None, what: str = "ShardedOptimizer") -> None:
    """Raises on EVERY rank of `group` unless all ranks hold the same `digest`.  A collective."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    seen = [None] * dist.get_world_size(group)
    dist.all_gather_object(seen, digest, group=group)
    if len(set(seen)) != 1:
        majority = max(set(seen), key=seen.count)
        odd = [r for r, d in enumerate(seen) if d != majority]
        raise RuntimeError(
            f"{what}: the ranks were given different parameter lists or options (ranks {odd} differ from the others); "
            "nothing was allocated or launched"
        )


class ShardedOptimizer:
    """Wraps one optimi_b200 (or any torch) optimizer class so that each rank steps 1/world of the elements.

    Args:
        optimizer_cls: the optimizer class, e.g. ``optimi_b200.AdamW``.
        params: tensors, or param-group dicts with per-group options.  Their storage is moved into
            flat buffers (one per dtype), values preserved.
        process_group: the ranks to shard over (default: the world group).
        split_on_tensors: cut ranges on tensor boundaries (set automatically for StableAdamW).
        gather: ``"nccl"`` (all-gather after the step) or a callable ``gather(flat, lo, hi)``.
        exchange: ``"nccl"``, ``"push"`` or ``"auto"`` (see the module docstring).
        reduce_grads: average the ranks' gradients inside the step kernel (push exchange only).
        pre_step_sync: push exchange: meet in a tiny collective before the step (see "Ordering").
        **kwargs: passed to the optimizer constructor.
    """

    def __init__(self, optimizer_cls: Callable, params, process_group=None, split_on_tensors: bool | None = None,
                 gather: str | Callable = "nccl", exchange: str = "nccl", reduce_grads: bool = False,
                 pre_step_sync: bool = True, **kwargs: Any):  # fmt: skip
        self.group = process_group
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        groups = _as_groups(params)
        self.params = [p for g in groups for p in g["params"]]
        if len({id(p) for p in self.params}) != len(self.params):
            raise ValueError("some parameters appear in more than one parameter group")
        if split_on_tensors is None:
            split_on_tensors = getattr(optimizer_cls, "__name__", "") == "StableAdamW"
        self.gather = gather
        can_push = (
            self.world > 1 and self.world <= 8 and hasattr(optimizer_cls, "_c_fn")
            and all(p.is_cuda for p in self.params) and len({p.device for p in self.params}) == 1
        )  # fmt: skip
        if exchange not in ("nccl", "push", "auto"):
            raise ValueError(f"unknown exchange mode {exchange!r}")
        if reduce_grads and split_on_tensors:
            raise ValueError("reduce_grads=True needs an optimizer other than StableAdamW")

        # every rank must be about to build the same layout; checked before anything is allocated or launched
        digest = layout_digest(groups, self.world, getattr(optimizer_cls, "__name__", str(optimizer_cls)), bool(split_on_tensors),
                               exchange, bool(reduce_grads), bool(can_push))  # fmt: skip
        assert_ranks_agree(digest, self.group)

        if exchange == "push" and not can_push:
            raise ValueError("exchange='push' needs 2-8 CUDA ranks on one device each and an optimi_b200 optimizer")
        self.exchange = "push" if (exchange in ("push", "auto") and can_push) else "nccl"
        if reduce_grads and self.exchange != "push":
            raise ValueError("reduce_grads=True needs the push exchange")
        self.reduce_grads = reduce_grads
        self.pre_step_sync = pre_step_sync
        self._peer_deltas: list[int] | None = None
        self._grad_deltas: list[int] | None = None
        self._symm_handles = []

        # one flat buffer per (device, dtype); under push all of them are regions of ONE symmetric allocation, so
        # that a single set of peer offsets serves every launch of the step
        by_dtype: dict[tuple, list[Tensor]] = {}
        group_index = {}
        for gi, g in enumerate(groups):
            for p in g["params"]:
                by_dtype.setdefault((p.device, p.dtype), []).append(p)
                group_index[id(p)] = gi
        layouts = {key: FlatLayout([p.numel() for p in plist], self.world, split_on_tensors) for key, plist in by_dtype.items()}
        region, arena_bytes = {}, 0
        for key, layout in layouts.items():
            region[key] = arena_bytes
            arena_bytes = _round_up(arena_bytes + layout.total * key[1].itemsize, ARENA_ALIGN)
        arena = grad_arena = None
        if self.exchange == "push":
            device = self.params[0].device
            arena, _, self._peer_deltas = self._symmetric_buffer(arena_bytes, device)
            if reduce_grads:
                grad_arena, _, others = self._symmetric_buffer(arena_bytes, device)
                others = iter(others)  # all ranks in rank order, 0 for this one
                self._grad_deltas = [0 if r == self.rank else next(others) for r in range(self.world)]

        self.buckets: list[dict[str, Any]] = []
        shards_of_group: list[list[Tensor]] = [[] for _ in groups]
        for key, plist in by_dtype.items():
            (device, dtype), layout = key, layouts[key]
            grad_flat = None
            if arena is not None:
                nbytes = layout.total * dtype.itemsize
                flat = arena[region[key] : region[key] + nbytes].view(dtype)
                if grad_arena is not None:
                    grad_flat = grad_arena[region[key] : region[key] + nbytes].view(dtype)
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
                shards_of_group[group_index[id(plist[i])]].append(sp)
            self.buckets.append(dict(layout=layout, flat=flat, params=plist, pieces=pieces, shards=shards, grad_flat=grad_flat))
        # the inner optimizer sees the same groups with the same options, holding this rank's pieces; its order of
        # parameters is group by group, which is the order `shard_params` keeps too
        self._groups = groups
        self._piece_of: dict[int, tuple[dict, tuple[int, int, int]]] = {}
        for b in self.buckets:
            for piece, sp in zip(b["pieces"], b["shards"]):
                self._piece_of[id(sp)] = (b, piece)
        self.shard_params = [sp for shards in shards_of_group for sp in shards]
        inner_groups = [{**{k: v for k, v in g.items() if k != "params"}, "params": shards} for g, shards in zip(groups, shards_of_group)]
        self.inner = optimizer_cls(inner_groups, **kwargs)
        if self.exchange == "push":
            self._meet = torch.zeros(1, dtype=torch.int32, device=self.params[0].device)
            # no rank may start pushing before every rank has finished filling its own buffer
            torch.cuda.synchronize(self.params[0].device)
            dist.barrier(self.group)

    def _symmetric_buffer(self, nbytes: int, device: torch.device):
        """A zeroed byte buffer every rank of the group can load from and store into: torch symmetric memory
        (CUDA virtual memory handles exchanged between the ranks); only plain peer loads and stores are
        used on it, by this package's own kernels.  Returns (buffer, handle, byte offsets from this rank's
        buffer to each peer's)."""
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        flat = symm.empty(nbytes, dtype=torch.uint8, device=device)
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
    def step_local(self, shard_grads: list[Tensor] | None = None, exchange: bool = True):
        """Steps this rank's range.  With the push exchange the step kernel also stores the updated
        parameters into the peers unless `exchange=False` (the local step alone: for measurements; the
        ranks' parameters then differ until a later exchanging step or `gather_params(force=True)`).
        `shard_grads`, one tensor per entry of `shard_params`, bypasses the parameters' `.grad` (a rank
        that received only its slice of the gradients from a reduce-scatter has nothing else)."""
        if shard_grads is None:
            self._bind_grads()
        else:
            for sp, g in zip(self.shard_params, shard_grads):
                sp.grad = g
        if self.exchange == "push" and exchange:
            from ._lib import peer_pull, peer_push

            if self.reduce_grads:
                if shard_grads is not None:
                    raise ValueError("reduce_grads=True reads the gradients of the shared buffer; do not pass shard_grads")
                dist.all_reduce(self._meet, group=self.group)  # every rank's gradients are written, nobody reads parameters any more
                self._init_states_from_mean_gradients()
                with peer_pull(self._grad_deltas, 1.0 / self.world), peer_push(self._peer_deltas):
                    self.inner.step()
            else:
                if self.pre_step_sync:
                    dist.all_reduce(self._meet, group=self.group)  # no peer still reads the parameters this step overwrites
                with peer_push(self._peer_deltas):
                    self.inner.step()
        else:
            if self.reduce_grads:
                raise ValueError("reduce_grads=True has no local-only step: the gradient mean exists only inside the fused kernel")
            self.inner.step()

    def _init_states_from_mean_gradients(self) -> None:
        """reduce_grads, first step only.  Some optimizers seed their state from the first gradient
        (Adan's previous gradient, SGD's `torch_init` momentum); the fused step never materialises the
        averaged gradient, so it is computed here once, with the kernel's own arithmetic (fp32 sum in
        rank order, times 1/world, one rounding), just for the state constructors.  The ranks' slices
        travel through an NCCL all-to-all into local memory; all arithmetic is on local tensors."""
        if getattr(self, "_states_seeded", False) or not hasattr(self.inner, "_init_state"):
            return
        self._states_seeded = True
        needs = getattr(self.inner, "_state_needs_first_gradient", None)
        if needs is None or not any(needs(g) for g in self.inner.param_groups):
            return
        group_of = {id(sp): g for g in self.inner.param_groups for sp in g["params"]}
        chunk = 1 << 24
        for b in self.buckets:
            layout, gf = b["layout"], b["grad_flat"]
            lo, hi = layout.rank_range(self.rank)
            per = hi - lo
            mean = torch.empty(per, dtype=gf.dtype, device=gf.device)
            for c0 in range(0, per, chunk):
                c1 = min(per, c0 + chunk)
                n = c1 - c0
                # slot r of `send` goes to rank r: this rank's gradients over rank r's range
                send = torch.cat([gf[layout.bounds[r] + c0 : layout.bounds[r] + c1] for r in range(self.world)])
                recv = torch.empty_like(send)
                dist.all_to_all_single(recv, send, group=self.group)
                acc = recv[:n].float()
                for r in range(1, self.world):
                    acc = acc + recv[r * n : (r + 1) * n].float()
                mean[c0:c1] = (acc * (1.0 / self.world)).to(gf.dtype)
            for (i, a, e), sp in zip(b["pieces"], b["shards"]):
                start = layout.offsets[i] + a - lo
                bound = sp.grad
                sp.grad = mean[start : start + e - a]
                self.inner._init_state(group_of[id(sp)], self.inner.state[sp], sp)
                sp.grad = bound
            del mean
        torch.cuda.synchronize()
        dist.barrier(self.group)

    @torch.no_grad()
    def gather_params(self, force: bool = False):
        """Hands every rank the updated parameters: one in-place all-gather per flat buffer.  With the push
        exchange the step kernel has already delivered them and only the closing meeting is left, unless
        `force=True` asks for the all-gather anyway (after `step_local(exchange=False)`)."""
        if self.world == 1:
            return
        if self.exchange == "push" and not force:
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

    # a step in pieces: begin_step(); step_groups([...]) as often as needed, each group once; end_step() -----
    @torch.no_grad()
    def begin_step(self, shard_grads: list[Tensor] | None = None) -> None:
        """Opens a step whose parameter groups are stepped one after another with `step_groups`, for gradients
        that arrive in pieces (copied in from the host, or reduced bucket by bucket): binds the gradients and,
        under the push exchange, holds the meeting that must precede the first pushing launch."""
        if self.reduce_grads:
            raise NotImplementedError("a step in pieces is not available with reduce_grads=True")
        if shard_grads is None:
            self._bind_grads()
        else:
            for sp, g in zip(self.shard_params, shard_grads):
                sp.grad = g
        if self.exchange == "push" and self.pre_step_sync:
            dist.all_reduce(self._meet, group=self.group)

    @torch.no_grad()
    def step_groups(self, indices) -> None:
        """Steps this rank's pieces of the parameter groups `indices` (pushing them to the peers under the push
        exchange).  Between `begin_step()` and `end_step()`; every group exactly once per step."""
        if not hasattr(self.inner, "step_groups"):
            raise NotImplementedError("step_groups needs an optimi_b200 optimizer")
        if self.exchange == "push":
            from ._lib import peer_push

            with peer_push(self._peer_deltas):
                self.inner.step_groups(indices)
        else:
            self.inner.step_groups(indices)

    @torch.no_grad()
    def end_step(self) -> None:
        """Closes a step in pieces: the exchange (all-gather, or the meeting that follows the pushes)."""
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

    # gradient clipping -------------------------------------------------------------------------
    @torch.no_grad()
    def clip_grad_norm(self, max_norm: float) -> Tensor:
        """The sharded form of `optimi_b200` optimizers' `clip_grad_norm`: each rank reads only the gradients
        of its own range, the ranks add up their per-tensor sums of squares (one small all-reduce), and
        every rank derives the same clip coefficient, which the next `step()` applies as it loads the
        gradients.  Returns the total norm (0-dim CUDA tensor).  Gradients must already be reduced across
        ranks: not available with `reduce_grads=True`, where the averaged gradient exists only inside the
        fused kernel."""
        if self.reduce_grads:
            raise NotImplementedError("clip_grad_norm needs materialised, already reduced gradients: not with reduce_grads=True")
        if not hasattr(self.inner, "_clip_from_sumsq"):
            raise NotImplementedError("clip_grad_norm needs an optimi_b200 optimizer")
        self._bind_grads()
        index_of = {id(p): i for i, p in enumerate(self.params)}
        owners = [index_of[id(self._piece_of[id(sp)][0]["params"][self._piece_of[id(sp)][1][0]])] for sp in self.shard_params]
        dtypes = [p.dtype for p in self.params]

        def reduce_sums(sumsq: Tensor) -> None:
            if self.world > 1:
                dist.all_reduce(sumsq, group=self.group)

        return self.inner._clip_from_sumsq(self.shard_params, owners, dtypes, float(max_norm), reduce_sums)

    # replica check -----------------------------------------------------------------------------
    @torch.no_grad()
    def replica_checksums(self) -> Tensor:
        """Integer checksums of this rank's copy of all parameters: the sum of the raw bit patterns of every
        `CHECKSUM_CHUNK` elements of each flat buffer, as int64 on the parameters' device."""
        sums = []
        for b in self.buckets:
            flat = b["flat"]
            bits = flat.view({1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[flat.element_size()])
            for a in range(0, bits.numel(), CHECKSUM_CHUNK):
                sums.append(bits[a : a + CHECKSUM_CHUNK].sum(dtype=torch.int64))
        return torch.stack(sums)

    @torch.no_grad()
    def check_replicas(self) -> dict[str, Any]:
        """Do all ranks hold bit-identical parameters?  Every rank checksums its whole parameter buffers and
        the ranks compare (element-wise MIN and MAX over ranks must coincide).  A collective; synchronises.
        Returns {"ranks_identical": bool, "bytes": bytes checksummed per rank, "chunks": number of checksums}."""
        mine = self.replica_checksums()
        lo, hi = mine.clone(), mine.clone()
        if self.world > 1:
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.group)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.group)
        nbytes = sum(b["flat"].numel() * b["flat"].element_size() for b in self.buckets)
        return {"ranks_identical": bool(torch.equal(lo, hi)), "bytes": nbytes, "chunks": int(mine.numel())}

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
        groups, first = [], 0
        for g_inner, g_full in zip(self.inner.param_groups, self._groups):
            n = len(g_full["params"])
            groups.append({k: v for k, v in g_inner.items() if k != "params"} | {"params": list(range(first, first + n))})
            first += n
        # parameters that never received a gradient have no state, as in an unsharded optimizer
        state = {i: st for i, st in state.items() if st}
        return {"state": state, "param_groups": groups}

    def load_consolidated_state_dict(self, sd: dict[str, Any]) -> None:
        """Loads an unsharded state dict (from `consolidated_state_dict`, from a plain optimizer of this
        package or from the reference): every rank keeps the slices of its own range."""
        inner_sd = self.inner.state_dict()
        index_of = {id(p): i for i, p in enumerate(self.params)}
        new_state = {}
        for j, sp in enumerate(self.shard_params):  # the inner optimizer numbers its parameters in this order
            b, (i, a, e) = self._piece_of[id(sp)]
            full_param = b["params"][i]
            full = sd["state"].get(index_of[id(full_param)])
            if full is None:
                continue
            entry = {}
            for k, v in full.items():
                if torch.is_tensor(v) and v.dim() > 0 and v.numel() == full_param.numel():
                    entry[k] = v.reshape(-1)[a:e].clone()
                else:
                    entry[k] = v.clone() if torch.is_tensor(v) else v
            new_state[j] = entry
        if len(sd["param_groups"]) != len(inner_sd["param_groups"]):
            raise ValueError(f"state dict has {len(sd['param_groups'])} parameter groups, this optimizer {len(inner_sd['param_groups'])}")
        groups = []
        for g_new, g_old, g_full in zip(sd["param_groups"], inner_sd["param_groups"], self._groups):
            if len(g_new["params"]) != len(g_full["params"]):
                raise ValueError("state dict parameter groups do not match this optimizer's (different number of parameters in a group)")
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
