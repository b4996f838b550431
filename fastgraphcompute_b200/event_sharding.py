"""Sharding of an event batch over the GPUs of one node (one process per GPU).

Row splits delimit independent events: the neighbour search never crosses a row split
(extensions/binned_select_knn_cpu.cpp:92-98,128 of the reference offsets every candidate
cell by the event's own cell block), the kNN gradient couples only points of one event and
the GravNet Linear layers act row-wise.  A batch therefore shards by event with no exchange
on the data path; only the final result gather is a collective (NCCL over NVLink when the
tensors live on GPUs, gloo for CPU tensors in tests).  The reference itself has no
multi-device code.

Typical use, every rank holding the same batch:

    part = partition_events(row_splits, world_size)
    idx, distsq = sharded_binned_select_knn(K, coords, row_splits)      # gathered on all ranks

`knn_fn` / `replace_fn` let tests run the orchestration on CPU ranks with a CPU stand-in
for the kernels; the defaults are this package's CUDA entry points.
"""
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass
class EventPartition:
    """Which events each rank processes.

    events[r]     : event numbers of rank r, ascending
    points[r]     : number of points of rank r
    """
    events: List[List[int]]
    points: List[int]

    @property
    def world_size(self):
        return len(self.events)


def partition_events(row_splits, world_size: int, weights: Optional[Sequence[float]] = None) -> EventPartition:
    """Greedy longest-processing-time assignment of whole events to ranks.

    Events are taken in order of decreasing weight (default: their point count) and each goes
    to the currently lightest rank; ties go to the lowest rank, so every rank computes the
    same table from the same row_splits.  Events with no points are assigned too (they cost
    nothing) so that every event has exactly one owner.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    rs = [int(v) for v in torch.as_tensor(row_splits).cpu().tolist()]
    if len(rs) < 1 or any(b < a for a, b in zip(rs[:-1], rs[1:])):
        raise ValueError("row_splits must be non-decreasing")
    sizes = [b - a for a, b in zip(rs[:-1], rs[1:])]
    if weights is None:
        weights = sizes
    if len(weights) != len(sizes):
        raise ValueError("one weight per event expected")
    order = sorted(range(len(sizes)), key=lambda e: (-float(weights[e]), e))
    load = [0.0] * world_size
    events = [[] for _ in range(world_size)]
    points = [0] * world_size
    for e in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        events[r].append(e)
        load[r] += float(weights[e])
        points[r] += sizes[e]
    for ev in events:
        ev.sort()
    return EventPartition(events, points)


def shard_rows(row_splits, events: Sequence[int], device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Global row ids (int64, concatenated event by event) and local row splits of a shard.

    Only the per-event starts and sizes (a few numbers) are prepared on the host; the row ids
    themselves are generated on ``device``:  row = position in the shard + (start of its event
    in the batch - start of its event in the shard)."""
    rs = [int(v) for v in torch.as_tensor(row_splits).cpu().tolist()]
    starts = [rs[e] for e in events]
    sizes = [rs[e + 1] - rs[e] for e in events]
    n_local = sum(sizes)
    local = torch.zeros(len(events) + 1, dtype=torch.int64)
    if events:
        local[1:] = torch.cumsum(torch.tensor(sizes, dtype=torch.int64), 0)
    dev = device if device is not None else torch.device("cpu")
    local = local.to(dev)
    if n_local == 0:
        return torch.zeros(0, dtype=torch.int64, device=dev), local
    shift = torch.tensor(starts, dtype=torch.int64, device=dev) - local[:-1]
    rows = torch.arange(n_local, dtype=torch.int64, device=dev) + torch.repeat_interleave(
        shift, torch.tensor(sizes, dtype=torch.int64, device=dev), output_size=n_local)
    return rows, local


def _default_knn():
    from .extensions.binned_select_knn import binned_select_knn
    return binned_select_knn


def _default_replace():
    from .extensions.index_replacer import index_replacer
    return index_replacer


def local_binned_select_knn(K, coords, row_splits, events, direction=None,
                            torch_compatible_indices=False, knn_fn: Optional[Callable] = None,
                            replace_fn: Optional[Callable] = None):
    """kNN of the given events only; returns (global_rows, idx with GLOBAL ids, distsq).

    The shard is searched with local row ids and mapped to global ids with index_replacer
    (-1 entries stay -1), the same op the reference uses to undo its own bin sort.
    """
    knn_fn = knn_fn or _default_knn()
    replace_fn = replace_fn or _default_replace()
    rows, local_rs = shard_rows(row_splits, events, device=coords.device)
    local_coords = coords.index_select(0, rows).contiguous()
    local_dir = None if direction is None else direction.index_select(0, rows).contiguous()
    idx, dsq = knn_fn(K, local_coords, local_rs, direction=local_dir,
                      torch_compatible_indices=torch_compatible_indices)
    return rows, replace_fn(idx.contiguous(), rows), dsq


def gather_rows(rows, tensors, n_total, points_per_rank, group=None):
    """All-gather per-rank row blocks into full tensors in global row order, on every rank.

    Contributions differ in length, so each rank pads to the largest shard; the receiver cuts
    the padding off using the partition table (known on every rank) and checks that it agrees
    with the sizes the ranks report.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_local = rows.shape[0]
    if n_local != points_per_rank[rank]:
        raise RuntimeError("shard of rank %d has %d rows, the partition table says %d"
                           % (rank, n_local, points_per_rank[rank]))
    sizes = torch.tensor([n_local], dtype=torch.int64, device=rows.device)
    all_sizes = [torch.zeros_like(sizes) for _ in range(world)]
    dist.all_gather(all_sizes, sizes, group=group)
    all_sizes = [int(s.item()) for s in all_sizes]
    if all_sizes != list(points_per_rank):
        raise RuntimeError("ranks disagree with the partition table: %s vs %s" % (all_sizes, list(points_per_rank)))
    if sum(all_sizes) != n_total:
        raise RuntimeError("shards do not cover the batch: %d rows of %d" % (sum(all_sizes), n_total))
    n_max = max(all_sizes) if all_sizes else 0

    def pad(t):
        if t.shape[0] == n_max:
            return t.contiguous()
        p = torch.zeros((n_max,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        p[: t.shape[0]] = t
        return p

    # one receive buffer per tensor ([world * n_max, ...], rank r's block at r * n_max): a single
    # collective each, no per-rank staging copies
    rows_all = torch.empty((world * n_max,), dtype=rows.dtype, device=rows.device)
    dist.all_gather_into_tensor(rows_all, pad(rows), group=group)
    outs = []
    for t in tensors:
        buf = torch.empty((world * n_max,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(buf, pad(t), group=group)
        full = torch.empty((n_total,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        for r in range(world):
            lo = r * n_max
            full.index_copy_(0, rows_all[lo: lo + all_sizes[r]], buf[lo: lo + all_sizes[r]])
        outs.append(full)
    return outs


def sharded_binned_select_knn(K, coords, row_splits, direction=None, torch_compatible_indices=False,
                              group=None, gather=True, knn_fn: Optional[Callable] = None,
                              replace_fn: Optional[Callable] = None):
    """binned_select_knn over a batch that every rank holds, each rank searching its own events.

    Returns (idx, distsq) for the whole batch on every rank (gather=True), or this rank's
    (global_rows, idx, distsq) block without any collective (gather=False).  Forward only.
    """
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    part = partition_events(row_splits, world)
    rows, idx, dsq = local_binned_select_knn(K, coords, row_splits, part.events[rank], direction,
                                             torch_compatible_indices, knn_fn, replace_fn)
    if not gather:
        return rows, idx, dsq
    full_idx, full_dsq = gather_rows(rows, [idx, dsq], coords.shape[0], part.points, group)
    return full_idx, full_dsq


def allreduce_gradients(parameters, group=None):
    """Sum the gradients of ``parameters`` over the ranks in ONE all-reduce.

    The exchange step of data-parallel training over event shards: every rank runs forward and
    backward on its own events (same module weights everywhere), the parameter gradients -- a
    few thousand floats for a GravNet layer -- are flattened into one buffer, summed over the
    ranks and written back, so that every rank holds the gradient of the whole batch.
    Parameters without a gradient count as zero."""
    params = [p for p in parameters]
    if not params:
        return
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).to(torch.float32)
                      for p in params])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    off = 0
    for p in params:
        n = p.numel()
        g = flat[off: off + n].view_as(p).to(p.dtype)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += n
