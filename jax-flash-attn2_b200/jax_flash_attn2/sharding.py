"""Partitioning of one attention call over the GPUs of a box.

The unit of work is one (batch element, key/value head): its group of query heads, one K head
and one V head. Units are independent in the forward and in the backward (dk / dv reduce only
inside a group), so every GPU runs the same single-GPU kernels on its slice and no collective
sits on the path. The reference has no counterpart: it relies on XLA to place its Triton custom
call (outputs inherit q's sharding, flash_attention_triton/_forward_triton.py:543) and offers a
device_put workaround (flash_attention.py:229-238) instead.
"""
from __future__ import annotations

import math
import typing as tp
from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    """Slice of the (batch, kv head) grid owned by one rank."""

    rank: int
    world_size: int
    batch_start: int
    batch_stop: int
    kv_head_start: int
    kv_head_stop: int

    @property
    def units(self) -> int:
        return (self.batch_stop - self.batch_start) * (self.kv_head_stop - self.kv_head_start)


def mesh_shape(batch: int, heads_kv: int, world_size: int) -> tp.Tuple[int, int]:
    """(ranks along batch, ranks along kv heads). Batch is split first; what is left of the world
    size splits the kv heads. Raises if the grid cannot be split evenly."""
    nb = math.gcd(batch, world_size)
    nh = world_size // nb
    if heads_kv % nh != 0:
        raise ValueError(
            f"cannot split batch={batch} x kv_heads={heads_kv} evenly over {world_size} ranks"
        )
    return nb, nh


def plan(batch: int, heads_kv: int, world_size: int, rank: int) -> Shard:
    nb, nh = mesh_shape(batch, heads_kv, world_size)
    rb, rh = divmod(rank, nh)
    pb, ph = batch // nb, heads_kv // nh
    return Shard(rank, world_size, rb * pb, (rb + 1) * pb, rh * ph, (rh + 1) * ph)


def slice_inputs(shard: Shard, group: int, q, k, v, *rest):
    """Views (no copies) of [B, S, H, D] tensors for this shard. `rest` are further tensors with
    query-head layout (o, dO, ...). Returns (q, k, v, *rest, kwargs) where kwargs carries the
    offsets that keep the dropout bits identical to the unsharded call."""
    b0, b1 = shard.batch_start, shard.batch_stop
    h0, h1 = shard.kv_head_start, shard.kv_head_stop
    qs = q[b0:b1, :, h0 * group:h1 * group]
    ks = k[b0:b1, :, h0:h1]
    vs = v[b0:b1, :, h0:h1]
    others = tuple(x[b0:b1, :, h0 * group:h1 * group] for x in rest)
    kwargs = dict(batch_offset=b0, head_offset=h0 * group, heads_q_global=q.shape[2])
    return (qs, ks, vs, *others, kwargs)


def max_over_ranks(value: float, device=None) -> float:
    """Largest `value` over all ranks of the default process group (the timing rule for anything
    measured on several GPUs); `value` itself when no process group is up."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_shards(shard: Shard, group: int, local: tp.Sequence, full_shapes: tp.Sequence[tp.Sequence[int]],
                  kv_layout: tp.Sequence[bool]):
    """Collects every rank's slices into full tensors on every rank (test and debugging aid; the
    product path never needs it: outputs stay where their shard ran). `local[i]` is this rank's
    slice of a [B, S, H, D] tensor whose full shape is `full_shapes[i]`; `kv_layout[i]` says
    whether its head axis counts key/value heads (k, v, dk, dv) or query heads."""
    import torch
    import torch.distributed as dist

    pieces = [None] * shard.world_size
    mine = (shard, [x.cpu() for x in local])
    if shard.world_size > 1:
        dist.all_gather_object(pieces, mine)
    else:
        pieces = [mine]
    full = [torch.zeros(tuple(shape), dtype=x.dtype) for shape, x in zip(full_shapes, local)]
    for sh, tensors in pieces:
        for dst, src, is_kv in zip(full, tensors, kv_layout):
            g = 1 if is_kv else group
            dst[sh.batch_start:sh.batch_stop, :, sh.kv_head_start * g:sh.kv_head_stop * g] = src
    return full
