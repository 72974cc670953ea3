"""Row sharding of the five hot-path ops across the GPUs of one box, and the output all-gather.

Upstream is single-device (``cuda_driver.py:292-300`` pins ordinal 0); this is the only multi-GPU
logic the b200 path needs.  Every op is embarrassingly parallel over one outer axis, so a rank owns a
contiguous slice of that axis, runs the ordinary single-GPU kernel on it, and the output slices are
all-gathered (NCCL over NVLink on GPUs; the same code runs over gloo on CPU for tests).  Inputs are
never exchanged: they are generated or delivered already sharded, B of a GEMM and the RMSNorm weight
are replicated.  ``torch`` is imported lazily so the package itself stays torch-free.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


def shard_bounds(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, near-equal split of ``range(total)``: the first ``total % world`` ranks get one extra."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    if total < 0:
        raise ValueError("total must be >= 0")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


@dataclass(frozen=True)
class ShardSpec:
    """Which axis of which argument positions a plan splits, and which arguments are replicated."""

    kind: str
    extent: int                       # length of the sharded outer axis
    sharded: tuple[tuple[int, int], ...]   # (argument position, axis)
    replicated: tuple[int, ...]
    outputs: tuple[int, ...]          # argument positions that are all-gathered afterwards
    # argument positions whose contents the kernel needs on the device before it runs: every tensor it reads, and
    # every output it only partly overwrites (a guarded or short store leaves the other elements as they were)
    reads: tuple[int, ...] = ()


def shard_spec(plan: Any, ir: Any) -> ShardSpec:
    """Sharding of a matched plan (see ``backend.matcher``): elementwise → flat chunks of axis 0, RMSNorm →
    rows, GEMM → M (A and C by rows, B replicated), attention → batch, LayerNorm → rows, reductions that keep
    the leading axis → rows (others do not shard)."""
    kind = plan.kind
    if kind == "elementwise":
        if plan.mode != "flat":
            raise ValueError("a body whose accesses are not one shared element-to-element map does not split along axis 0")
        tensors = tuple(dict.fromkeys(tuple(plan.inputs) + tuple(store[0] for store in plan.stores)))
        shapes = {ir.arguments[p].spec.shape for p in tensors}
        if len(shapes) != 1:
            raise ValueError("elementwise sharding needs tensors of one shape")
        shape = next(iter(shapes))
        # operands read by address arithmetic (a one-element tensor used as a scalar, a row vector broadcast over the
        # rows) are the same for every shard; one that varies along the split axis would have to be split with it
        gathers = tuple(getattr(plan, "gathers", ()))
        for node in plan.nodes:
            if node.op == "broadcast_input" and node.attrs["source_shape"][0] != 1:
                raise ValueError("an operand broadcast along the columns varies along the shard axis; this kernel does not shard")
        stored = tuple(store[0] for store in plan.stores)
        numel = 1
        for length in shape:
            numel *= length
        partly = stored if plan.extent < numel else ()
        return ShardSpec(kind, shape[0], tuple((p, 0) for p in tensors), gathers, stored,
                         reads=tuple(dict.fromkeys(tuple(plan.inputs) + gathers + partly)))
    if kind == "rmsnorm":
        full = (plan.gamma,) if plan.gamma_is_full else ()
        shape = ir.arguments[plan.x].spec.shape
        if len(shape) < 2:
            raise ValueError("a rank-1 rmsnorm has a single row and does not shard")
        return ShardSpec(kind, shape[0], tuple((p, 0) for p in (plan.x, plan.out) + full),
                         () if plan.gamma_is_full else (plan.gamma,), (plan.out,), reads=(plan.x, plan.gamma))
    if kind == "gemm":
        a_axis = 1 if plan.transpose_a else 0  # A is [m,k] or, transposed, [k,m]
        return ShardSpec(kind, plan.m, ((plan.a, a_axis), (plan.c, 0)), (plan.b,), (plan.c,), reads=(plan.a, plan.b))
    if kind == "attention":
        return ShardSpec(kind, plan.batch, tuple((p, 0) for p in (plan.q, plan.k, plan.v, plan.out, plan.lse)), (),
                         (plan.out, plan.lse), reads=(plan.q, plan.k, plan.v))
    if kind == "layernorm":
        shape = ir.arguments[plan.x].spec.shape
        if len(shape) < 2:
            raise ValueError("a rank-1 layernorm has a single row and does not shard")
        per_row = (plan.x, plan.residual, plan.out, plan.out_resid)
        full = tuple(p for p, is_full in ((plan.weight, plan.weight_is_full), (plan.bias, plan.bias_is_full)) if is_full)
        shared = tuple(p for p, is_full in ((plan.weight, plan.weight_is_full), (plan.bias, plan.bias_is_full)) if not is_full)
        return ShardSpec(kind, shape[0], tuple((p, 0) for p in per_row + full), shared, (plan.out, plan.out_resid),
                         reads=(plan.x, plan.residual, plan.weight, plan.bias))
    if kind == "reduction_bundle":
        raise ValueError("a bundle of reductions folds over different axes of one tensor; it does not shard")
    if kind == "reduction":
        # only a fold that keeps the leading axis splits without an exchange step (each rank folds its own rows);
        # folds over the leading axis run whole on one GPU
        if plan.form == "rows" and len(plan.source_shape) >= 2 and ir.arguments[plan.dst].spec.shape[:1] == plan.source_shape[:1]:
            return ShardSpec(kind, plan.source_shape[0], tuple((p, 0) for p in tuple(plan.inputs) + (plan.dst,)), (), (plan.dst,),
                             reads=tuple(plan.inputs))
        # a scalar result lands at one offset of dst: the rest of dst keeps its contents
        return ShardSpec(kind, 1, (), tuple(plan.inputs) + (plan.dst,), (plan.dst,), reads=tuple(plan.inputs) + (plan.dst,))
    raise ValueError(f"unknown plan kind '{kind}'")


def local_slices(spec: ShardSpec, world: int, rank: int) -> dict[int, tuple[int, slice]]:
    """argument position → (axis, slice) this rank owns."""
    start, stop = shard_bounds(spec.extent, world, rank)
    return {position: (axis, slice(start, stop)) for position, axis in spec.sharded}


def all_gather_rows(local, group=None):
    """All-gather equal-or-ragged row shards of a tensor along axis 0 into one tensor on every rank."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if world == 1:
        return local
    rows = torch.tensor([local.shape[0]], device=local.device, dtype=torch.int64)
    counts = [torch.zeros_like(rows) for _ in range(world)]
    dist.all_gather(counts, rows, group=group)
    counts = [int(c.item()) for c in counts]
    if len(set(counts)) == 1:
        gathered = torch.empty((world * counts[0],) + tuple(local.shape[1:]), device=local.device, dtype=local.dtype)
        dist.all_gather_into_tensor(gathered, local.contiguous(), group=group)
        return gathered
    # ragged shards: pad to the longest, gather equal-sized pieces, trim
    longest = max(counts)
    padded = torch.zeros((longest,) + tuple(local.shape[1:]), device=local.device, dtype=local.dtype)
    padded[: local.shape[0]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    return torch.cat([piece[:count] for piece, count in zip(pieces, counts)], dim=0)


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Device-time reduction used for every multi-GPU number: the slowest rank defines the step."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    cell = torch.tensor([float(value)], device=device or "cpu", dtype=torch.float64)
    dist.all_reduce(cell, op=dist.ReduceOp.MAX, group=group)
    return float(cell.item())
