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


def chunk_events(events: Sequence[int], row_splits, n_chunks: int) -> List[List[int]]:
    """Split one rank's (ascending) event list into ``n_chunks`` consecutive groups of about the
    same number of points; groups may be empty.  A pure function of its arguments, so every rank
    computes every other rank's groups from the partition table alone."""
    rs = [int(v) for v in torch.as_tensor(row_splits).cpu().tolist()]
    n_chunks = max(int(n_chunks), 1)
    sizes = [rs[e + 1] - rs[e] for e in events]
    total = sum(sizes)
    out = [[] for _ in range(n_chunks)]
    acc = 0
    for e, sz in zip(events, sizes):
        # the group in which the event's midpoint falls
        c = min(n_chunks - 1, int((acc + 0.5 * sz) * n_chunks / total)) if total > 0 else 0
        out[c].append(e)
        acc += sz
    return out


def _agree_or_raise(ok: bool, message: str, device, group=None):
    """All ranks learn whether every rank is ready to exchange; a rank that is not raises its own
    message, the others raise a generic one -- before any data moves, so that nobody waits for a
    peer that has left."""
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if not ok:
        raise RuntimeError(message)
    if int(flag.item()) == 0:
        raise RuntimeError("another rank's shard disagrees with the partition table; nothing was exchanged")


class EventRowExchange:
    """Moves per-event row blocks of the ranks into full tensors in global row order.

    Events are contiguous row ranges of the batch, so a block is sent from the owner's local
    result straight into rows [row_splits[e], row_splits[e+1]) of the receiver's full tensor: no
    padding, no staging buffer, no re-ordering pass.  One grouped set of point-to-point transfers
    per call of ``post`` (NCCL over NVLink for CUDA tensors, gloo on CPU); the transfers of one
    group of events can run while the next group is still being searched.

    mode "all": every rank receives every block; "root": only ``root`` does.
    """

    def __init__(self, row_splits, part: EventPartition, templates, mode="all", root=0, group=None):
        if mode not in ("all", "root"):
            raise ValueError("mode must be 'all' or 'root'")
        self.rs = [int(v) for v in torch.as_tensor(row_splits).cpu().tolist()]
        self.part = part
        self.mode = mode
        self.root = root
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.receives = mode == "all" or self.rank == root
        n_total = self.rs[-1]
        # templates: (dtype, trailing shape, device) per exchanged tensor
        self.full = [torch.empty((n_total,) + tuple(shape), dtype=dtype, device=device) if self.receives else None
                     for dtype, shape, device in templates]
        self.pending = []
        self.keep = []
        self.groups = []          # per post(): (works, row ranges of every rank's events, event after the own-row copies)
        self.comm_stream = None
        dev = templates[0][2]
        if torch.device(dev).type == "cuda":
            self.comm_stream = torch.cuda.Stream(device=dev)

    def _global_rank(self, r):
        return r if self.group is None else dist.get_global_rank(self.group, r)

    def post(self, my_events: Sequence[int], blocks, events_of_rank):
        """Start the transfers of one group: ``blocks`` are this rank's tensors for ``my_events``
        (rows concatenated event by event), ``events_of_rank[r]`` the events rank r contributes
        in this group.  Returns at once; ``finish`` waits."""
        sizes = [self.rs[e + 1] - self.rs[e] for e in my_events]
        n_local = sum(sizes)
        for b in blocks:
            if b.shape[0] != n_local:
                raise RuntimeError("shard of rank %d has %d rows, the partition table says %d"
                                   % (self.rank, b.shape[0], n_local))
        ops = []
        peers = [p for p in range(self.world) if p != self.rank]
        # own rows: a device copy per event
        if self.receives:
            off = 0
            for e, sz in zip(my_events, sizes):
                for full, b in zip(self.full, blocks):
                    full[self.rs[e]: self.rs[e] + sz].copy_(b[off: off + sz], non_blocking=True)
                off += sz
        for p in peers:
            if self.mode == "all" or p == self.root:
                off = 0
                for e, sz in zip(my_events, sizes):
                    if sz:
                        for b in blocks:
                            ops.append(dist.P2POp(dist.isend, b[off: off + sz], self._global_rank(p), self.group))
                    off += sz
            if self.receives:
                for e in events_of_rank[p]:
                    sz = self.rs[e + 1] - self.rs[e]
                    if sz:
                        for full in self.full:
                            ops.append(dist.P2POp(dist.irecv, full[self.rs[e]: self.rs[e] + sz],
                                                  self._global_rank(p), self.group))
        self.keep.append(blocks)
        ranges = []
        if self.receives:
            for r in range(self.world):
                for e in events_of_rank[r]:
                    if self.rs[e + 1] > self.rs[e]:
                        ranges.append((self.rs[e], self.rs[e + 1]))
        copied = None
        if self.comm_stream is not None:
            copied = torch.cuda.Event()
            copied.record(torch.cuda.current_stream(self.comm_stream.device))
        works = []
        if ops:
            if self.comm_stream is not None:
                # issue from a side stream that waits for the producer of the blocks: the launching
                # stream is free to start the next group's search while these transfers run
                self.comm_stream.wait_stream(torch.cuda.current_stream(self.comm_stream.device))
                with torch.cuda.stream(self.comm_stream):
                    works = dist.batch_isend_irecv(ops)
            else:
                works = dist.batch_isend_irecv(ops)
        self.pending.extend(works)
        self.groups.append((works, ranges, copied))

    def wait_group(self, i, stream=None):
        """Make ``stream`` (CUDA; on CPU: the caller) wait until the rows of the i-th posted group
        are in the full tensors -- the transfers and this rank's own copies -- and return their
        row ranges [(begin, end), ...].  Lets a caller work on a finished group (widen its ids)
        while later groups are still searched or in flight."""
        works, ranges, copied = self.groups[i]
        if stream is not None:
            with torch.cuda.stream(stream):
                for w in works:
                    w.wait()
            if copied is not None:
                stream.wait_event(copied)
        else:
            for w in works:
                w.wait()
            # (host waits are final: finish() must not wait for these a second time)
            done = set(id(w) for w in works)
            self.pending = [w for w in self.pending if id(w) not in done]
        return ranges

    def finish(self):
        """Wait for every posted transfer; returns the full tensors (None on a rank that does not
        receive)."""
        if self.comm_stream is not None:
            with torch.cuda.stream(self.comm_stream):
                for w in self.pending:
                    w.wait()
            torch.cuda.current_stream(self.comm_stream.device).wait_stream(self.comm_stream)
        else:
            for w in self.pending:
                w.wait()
        self.pending = []
        self.keep = []
        self.groups = []
        return self.full


def gather_rows(rows, tensors, n_total, points_per_rank, group=None, row_splits=None, part=None,
                mode="all", root=0):
    """Bring per-rank row blocks (rows of the rank's events, event by event) together as full
    tensors in global row order: on every rank (mode "all") or on ``root`` only (mode "root",
    other ranks get None).  The ranks first agree that every shard has the size the partition
    table says (one 4-byte all-reduce and a host read); a rank whose shard differs raises, and so
    do the others, before any row moves."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_local = rows.shape[0]
    ok = n_local == points_per_rank[rank] and sum(points_per_rank) == n_total
    _agree_or_raise(ok, "shard of rank %d has %d rows, the partition table says %d (batch: %d rows, table: %d)"
                    % (rank, n_local, points_per_rank[rank], n_total, sum(points_per_rank)), rows.device, group)
    if row_splits is None or part is None:
        raise ValueError("gather_rows needs the row splits and the partition table")
    ex = EventRowExchange(row_splits, part, [(t.dtype, t.shape[1:], t.device) for t in tensors], mode, root, group)
    ex.post(part.events[rank], [t.contiguous() for t in tensors], part.events)
    return ex.finish()


def _gather_all_collective(K, coords, row_splits, chunks, search, group, rank, world):
    """Rows of every rank on every rank through one all-gather per group of events.

    The partition balances the ranks' row counts to a fraction of a per cent, so padding every
    rank's block of a group to the largest one costs next to nothing, and an all-gather moves the
    same bytes at the collective's bandwidth (NCCL rings / NVSwitch) where grouped point-to-point
    transfers reached about half of it.  Every rank then has all blocks in shard order in a staging
    buffer of its own memory; one pass per event places the rows at their global positions and
    widens the ids to int64 (the pass the ids need anyway).  Group c is in flight while group c+1
    is searched and group c-1 is placed."""
    rs = [int(v) for v in torch.as_tensor(row_splits).cpu().tolist()]
    n_total = rs[-1]
    dev = coords.device
    cuda = dev.type == "cuda"
    full_idx = torch.empty((n_total, K), dtype=torch.int64, device=dev)
    full_dsq = torch.empty((n_total, K), dtype=torch.float32, device=dev)
    comm_stream = torch.cuda.Stream(device=dev) if cuda else None
    place_stream = torch.cuda.Stream(device=dev) if cuda else None
    groups = []

    def place(g):
        works, staged_i, staged_d, m, c = g[:5]
        ctx = torch.cuda.stream(place_stream) if cuda else None
        if ctx is not None:
            ctx.__enter__()
        try:
            for w in works:
                w.wait()
            for r in range(world):
                off = r * m
                for e in chunks[r][c]:
                    sz = rs[e + 1] - rs[e]
                    if sz:
                        full_idx[rs[e]: rs[e] + sz].copy_(staged_i[off: off + sz], non_blocking=True)
                        full_dsq[rs[e]: rs[e] + sz].copy_(staged_d[off: off + sz], non_blocking=True)
                    off += sz
        finally:
            if ctx is not None:
                ctx.__exit__(None, None, None)

    n_groups = len(chunks[rank])
    for c in range(n_groups):
        rows_of = [sum(rs[e + 1] - rs[e] for e in chunks[r][c]) for r in range(world)]
        m = max(rows_of)
        if m == 0:
            groups.append(None)
            continue
        send_i = torch.empty((m, K), dtype=torch.int32, device=dev)
        send_d = torch.empty((m, K), dtype=torch.float32, device=dev)
        mine = chunks[rank][c]
        if mine:
            _, idx, dsq = search(mine)
            if idx.shape[0] != rows_of[rank]:
                raise RuntimeError("shard of rank %d has %d rows, the partition table says %d"
                                   % (rank, idx.shape[0], rows_of[rank]))
            send_i[: idx.shape[0]].copy_(idx)
            send_d[: idx.shape[0]].copy_(dsq)
        staged_i = torch.empty((world * m, K), dtype=torch.int32, device=dev)
        staged_d = torch.empty((world * m, K), dtype=torch.float32, device=dev)
        if cuda:
            comm_stream.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(comm_stream):
                works = [dist.all_gather_into_tensor(staged_i, send_i, group=group, async_op=True),
                         dist.all_gather_into_tensor(staged_d, send_d, group=group, async_op=True)]
        else:
            works = [dist.all_gather_into_tensor(staged_i, send_i, group=group, async_op=True),
                     dist.all_gather_into_tensor(staged_d, send_d, group=group, async_op=True)]
        groups.append((works, staged_i, staged_d, m, c, send_i, send_d))
        if c > 0 and groups[c - 1] is not None:
            place(groups[c - 1])
    if groups and groups[-1] is not None:
        place(groups[-1])
    if cuda:
        torch.cuda.current_stream(dev).wait_stream(place_stream)
        torch.cuda.current_stream(dev).wait_stream(comm_stream)
    return full_idx, full_dsq


def sharded_binned_select_knn(K, coords, row_splits, direction=None, torch_compatible_indices=False,
                              group=None, gather=True, knn_fn: Optional[Callable] = None,
                              replace_fn: Optional[Callable] = None, root=0, n_chunks=1, check=True,
                              exchange="auto"):
    """binned_select_knn over a batch that every rank holds, each rank searching its own events.

    gather = True / "all": (idx, distsq) of the whole batch on every rank; "root": on ``root``
    only (None, None elsewhere); False / "none": this rank's (global_rows, idx, distsq) block
    without any collective.  Forward only.

    Neighbour ids travel as int32 (row counts are below 2^31) and are widened to the public int64
    on receipt: a third fewer bytes on the links.  With n_chunks > 1 a rank searches its events
    in that many groups and the rows of a finished group travel while the next one is searched.
    check=False skips the agreement step (a 4-byte all-reduce and a host read).
    exchange: how the rows reach every rank with gather="all" -- "collective" (one all-gather per
    group into a staging buffer, then a placing pass; the default, "auto") or "p2p" (per-event
    point-to-point blocks straight into the final tensors, which is what gather="root" always uses).
    """
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    mode = {True: "all", False: "none"}.get(gather, gather)
    if mode not in ("all", "root", "none"):
        raise ValueError("gather must be True/'all', 'root' or False/'none'")
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    part = partition_events(row_splits, world)
    if mode == "none":
        return local_binned_select_knn(K, coords, row_splits, part.events[rank], direction,
                                       torch_compatible_indices, knn_fn, replace_fn)
    if check:
        n_total = int(torch.as_tensor(row_splits)[-1])
        _agree_or_raise(sum(part.points) == n_total == coords.shape[0],
                        "rank %d: the partition table covers %d rows, the batch has %d"
                        % (rank, sum(part.points), coords.shape[0]), coords.device, group)
    chunks = [chunk_events(part.events[r], row_splits, n_chunks) for r in range(world)]
    if exchange not in ("auto", "collective", "p2p"):
        raise ValueError("exchange must be 'auto', 'collective' or 'p2p'")
    if mode == "all" and exchange in ("auto", "collective"):
        def search(events):
            return local_binned_select_knn(K, coords, row_splits, events, direction, torch_compatible_indices,
                                           knn_fn, replace_fn)
        return _gather_all_collective(K, coords, row_splits, chunks, search, group, rank, world)
    ex = EventRowExchange(row_splits, part, [(torch.int32, (K,), coords.device), (torch.float32, (K,), coords.device)],
                          mode, root, group)
    # the public ids are int64: a finished group is widened on a stream of its own while the
    # next group is searched and in flight
    full_idx = None
    widen_stream = None
    if ex.receives:
        full_idx = torch.empty((ex.rs[-1], K), dtype=torch.int64, device=coords.device)
        if coords.is_cuda:
            widen_stream = torch.cuda.Stream(device=coords.device)

    def widen(i):
        if full_idx is None:
            return
        ranges = ex.wait_group(i, widen_stream)
        if widen_stream is not None:
            with torch.cuda.stream(widen_stream):
                for a, b in ranges:
                    full_idx[a:b].copy_(ex.full[0][a:b], non_blocking=True)
        else:
            for a, b in ranges:
                full_idx[a:b].copy_(ex.full[0][a:b])

    n_groups = max(int(n_chunks), 1)
    for c in range(n_groups):
        mine = chunks[rank][c]
        if mine:
            rows, idx, dsq = local_binned_select_knn(K, coords, row_splits, mine, direction,
                                                     torch_compatible_indices, knn_fn, replace_fn)
            blocks = [idx.to(torch.int32), dsq.contiguous()]
        else:
            blocks = [torch.empty((0, K), dtype=torch.int32, device=coords.device),
                      torch.empty((0, K), dtype=torch.float32, device=coords.device)]
        ex.post(mine, blocks, [chunks[r][c] for r in range(world)])
        if c > 0:
            widen(c - 1)
    widen(n_groups - 1)
    full_idx32, full_dsq = ex.finish()
    if full_idx32 is None:
        return None, None
    if widen_stream is not None:
        torch.cuda.current_stream(coords.device).wait_stream(widen_stream)
        full_idx32.record_stream(widen_stream)
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
