"""binned_select_knn -- drop-in for fastgraphcompute.extensions.binned_select_knn.

Same call signature, returned tensors and autograd behaviour as the reference
(extensions/binned_select_knn.py:12-94 on top of BinnedKNNAutograd,
extensions/binned_knn_autograd_kernel.cpp:84-253): indices int64 [N,K] with the
point itself in slot 0 and -1 in unused slots, squared distances float32 [N,K],
differentiable w.r.t. the coordinates through the distances only.
"""
import ctypes
import threading
from typing import Optional, Tuple

import torch

from .. import _cabi

# Mean number of points per search-grid cell the library aims for (<= 0: built-in default).
target_occupancy = 0.0
# Read the device status word after every forward (one small device->host copy).
# The reference synchronises several times per call; switching this off makes the
# call fully asynchronous but turns bad inputs (NaN, malformed row_splits) into
# silently unwritten outputs.
check_status = True
# Backward by sorted-segment reductions over a reverse neighbour graph instead of float atomics:
# bit-identical gradients from run to run (the atomic version, like the reference's CUDA path,
# sums in arrival order).  Falls back to the atomic kernel when N*K >= 2^31.
deterministic_backward = False


def _raise_for_status(status):
    if status & _cabi.STATUS_NONFINITE:
        raise RuntimeError("BinByCoordinates: input coordinates contain non-finite values")
    if status & _cabi.STATUS_BAD_ROW_SPLITS:
        raise RuntimeError("binned_select_knn: row_splits must start at 0, be non-decreasing and "
                           "end at the number of points (bin boundaries do not match row splits)")
    if status:
        raise RuntimeError("binned_select_knn: internal error, status %d" % status)


# D = 4 only.  The library chooses on the device between a grid over four coordinates and one
# over three (strongly clustered data) -- a trial histogram and a search kernel that holds both
# searches.  With grid_dims = 0 the wrapper remembers the last choice per device and asks for it
# directly on the following calls of the same shape (same device, point count, row-split count
# and K: no trial, the single-search kernel; C2: 1.07 -> 1.02 ms per forward + backward),
# returning to the automatic choice every `grid_probe_every` calls so that data whose character
# changes is noticed.  3 or 4 fix the form; -1 always lets the device choose.
# The neighbour sets never depend on the grid; only speed (and the slot order inside a row) does.
# Needs check_status (that is where the choice comes back to the host).
grid_dims = 0
grid_probe_every = 64
pad_min_pairs = 1 << 19    # backward for D = 3, 5, 6, 7: pad to four / eight coordinates from this many (row, slot) pairs on
_grid_memory = {}        # (device, N, row splits, K) -> [form, calls since the last automatic choice]
# forward calls may come from several host threads (one per stream or device) and the backward runs
# on autograd's own threads: the two module-level tables are only touched under this lock
_tables_lock = threading.Lock()


def knn_forward_raw(coords, row_splits, K, direction, tf_compat, count_evals=False):
    """Launch the forward (fgc_knn_build_grid + fgc_knn_search, which is what
    fgc_binned_knn_fwd does) on prepared tensors; returns (idx, distsq, workspace)."""
    dev = coords.device
    n_vert, n_coords = coords.shape
    n_rs = row_splits.numel()
    idx = torch.empty((n_vert, K), dtype=torch.int64, device=dev)
    dist = torch.empty((n_vert, K), dtype=torch.float32, device=dev)
    nbytes = _cabi.lib.fgc_knn_workspace_bytes(n_vert, n_coords, n_rs, K)
    if nbytes == 0:
        if K < 1 or K > _cabi.FGC_MAX_K:
            raise ValueError("binned_select_knn: K must be in 1..%d, got %d" % (_cabi.FGC_MAX_K, K))
        raise ValueError("binned_select_knn: unsupported problem size")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        stream = _cabi.current_stream(dev)
        form = 0
        if n_coords == 4:
            if grid_dims in (3, 4):
                form = grid_dims
            elif grid_dims == 0 and check_status:
                with _tables_lock:
                    mem = _grid_memory.get((dev.index, n_vert, n_rs, K))
                    if mem is not None and mem[1] < grid_probe_every:
                        form = mem[0]
                        mem[1] += 1
        _cabi.check(_cabi.lib.fgc_knn_build_grid_dims(
            _cabi.ptr(coords), n_vert, n_coords, _cabi.ptr(row_splits), n_rs, K,
            _cabi.ptr(direction), float(target_occupancy), form, _cabi.ptr(ws), nbytes, stream),
            "fgc_knn_build_grid_dims")
        status_host = None
        if check_status:
            # The status word is final once the grid is built (non-finite input and malformed
            # row_splits are detected by its first two kernels).  A one-thread kernel stores it
            # into pinned host memory now and the host looks at it after the search has been
            # launched: the host waits for the short grid build only, the GPU never idles while
            # the host checks, and -- unlike a device-to-host copy -- the store does not queue
            # behind bulk result copies that other streams have in flight.
            status_host = torch.empty(2, dtype=torch.int32, pin_memory=True)
            _cabi.check(_cabi.lib.fgc_knn_publish_grid_info(_cabi.ptr(ws), status_host.data_ptr(), stream),
                        "fgc_knn_publish_grid_info")
            status_ready = torch.cuda.Event()
            status_ready.record()
        _cabi.check(_cabi.lib.fgc_knn_search(
            n_vert, n_coords, n_rs, K, int(direction is not None), int(bool(tf_compat)),
            (1 if count_evals else 0) | (8 if form == 3 else 16 if form == 4 else 0) | 32,   # 32: first search of this grid
            _cabi.ptr(idx), _cabi.ptr(dist),
            _cabi.ptr(ws), nbytes, stream), "fgc_knn_search")
        if status_host is not None:
            status_ready.synchronize()
            info = status_host.tolist()
            _raise_for_status(int(info[0]))
            if n_coords == 4 and form == 0 and grid_dims == 0:
                with _tables_lock:
                    if len(_grid_memory) > 256:
                        _grid_memory.clear()
                    _grid_memory[(dev.index, n_vert, n_rs, K)] = [int(info[1]) & 15, 0]      # what the device chose
    return idx, dist, ws


def read_counters(ws):
    """(counters [8], grid shape [3], cell width) of a forward's workspace; counters[0] is the
    number of distance evaluations of a search launched with count_evals."""
    counters = (ctypes.c_uint64 * 8)()
    shape = (ctypes.c_int32 * 3)()
    width = ctypes.c_float(0)
    with torch.cuda.device(ws.device):
        _cabi.check(_cabi.lib.fgc_knn_read_counters(
            _cabi.ptr(ws), counters, shape, ctypes.byref(width),
            _cabi.current_stream(ws.device)), "fgc_knn_read_counters")
    return list(counters), [shape[0], shape[1], shape[2]], width.value


def cell_order(ws, n_vert, n_coords, n_rs, K):
    """int32 [n_vert] view into a forward's workspace: original ids in cell order (a permutation
    that keeps spatial neighbours together; used as processing order by the GravNet kernels)."""
    base = ws.data_ptr()
    p = _cabi.lib.fgc_knn_cell_order(_cabi.ptr(ws), n_vert, n_coords, n_rs, K)
    if not p:
        raise RuntimeError("fgc_knn_cell_order: bad arguments")
    off = p - base
    return ws[off:off + 4 * n_vert].view(torch.int32)


# One reverse-neighbour graph per neighbour-index tensor, shared by the deterministic backward
# passes that scatter through it (GravNet aggregation first, then the kNN distances): the entry
# keeps the index tensor alive, so its address cannot be reused while the entry exists, and
# the kNN backward -- the last consumer in a GravNet layer -- drops it.
_rgraph_cache = {}


def clear_reverse_graph_cache():
    with _tables_lock:
        _rgraph_cache.clear()


def reverse_graph(idx, keep):
    """Reverse-neighbour graph workspace of ``idx`` ([N, K] int64, contiguous) and its size in
    bytes; built by fgc_build_reverse_graph unless the previous caller left one for this very
    tensor.  ``keep``: leave it for the next caller (at most one graph is kept)."""
    n_vert, K = idx.shape
    stream = _cabi.current_stream(idx.device)
    key = (idx.data_ptr(), idx._version, n_vert, K, idx.device, getattr(stream, "value", stream))
    with _tables_lock:
        hit = _rgraph_cache.pop(key, None)
        _rgraph_cache.clear()
    if hit is not None:
        rg = hit[1]
    else:
        rbytes = _cabi.lib.fgc_reverse_graph_bytes(n_vert, K)
        if not rbytes:
            return None, 0
        rg = torch.empty(rbytes, dtype=torch.uint8, device=idx.device)
        _cabi.check(_cabi.lib.fgc_build_reverse_graph(
            _cabi.ptr(idx), n_vert, K, _cabi.ptr(rg), rbytes, stream), "fgc_build_reverse_graph")
    if keep:
        with _tables_lock:
            _rgraph_cache[key] = (idx, rg)
    return rg, rg.numel()


def knn_backward_raw(grad_dist, idx, coords, order=None):
    """Launch the backward (atomic or sorted-segment variant) on prepared tensors.  order: the
    forward's cell order (int32 [N]) as processing order of the atomic variant, or None."""
    n_vert, n_coords = coords.shape
    K = idx.shape[1]
    if n_coords in (3, 5, 6, 7) and not deterministic_backward and n_vert * K >= pad_min_pairs:
        # Rows of 12, 20, 24 or 28 bytes allow neither 16-byte gathers nor vector reductions: at
        # size, run the four- / eight-coordinate kernel on a zero-padded copy (the padded
        # differences are 0 and add nothing to a sum that is returned) and drop the padding
        # again.  Same arithmetic on the real coordinates; one or two 16-byte gathers and vector
        # reductions per neighbour instead of D of each (D = 3, 1.66 M rows, K = 64: 2.11 -> 0.98 ms).
        width = 4 if n_coords == 3 else 8
        padded = torch.zeros((n_vert, width), dtype=coords.dtype, device=coords.device)
        padded[:, :n_coords] = coords
        return knn_backward_raw(grad_dist, idx, padded, order)[:, :n_coords].contiguous()
    out = torch.empty_like(coords)
    with torch.cuda.device(coords.device):
        stream = _cabi.current_stream(coords.device)
        rg, rbytes = reverse_graph(idx, keep=False) if deterministic_backward else (None, 0)
        if rbytes:
            _cabi.check(_cabi.lib.fgc_binned_knn_bwd_sorted(
                _cabi.ptr(grad_dist), _cabi.ptr(idx), _cabi.ptr(coords), n_vert, K, n_coords,
                _cabi.ptr(rg), rbytes, _cabi.ptr(out), stream), "fgc_binned_knn_bwd_sorted")
        else:
            _cabi.check(_cabi.lib.fgc_binned_knn_bwd_ordered(
                _cabi.ptr(grad_dist), _cabi.ptr(idx), _cabi.ptr(coords), n_vert, K,
                n_coords, _cabi.ptr(order), _cabi.ptr(out), stream), "fgc_binned_knn_bwd_ordered")
    return out


class _BinnedKNN(torch.autograd.Function):
    """Eager-mode autograd node (the dispatcher op fgc_b200::knn_forward does the same for
    TorchScript and tracing; calling the library directly saves the dispatcher's Python
    round trips, about 0.1 ms per forward + backward)."""

    @staticmethod
    def forward(ctx, coords, row_splits, K, direction, tf_compat):
        _cabi.require_cuda(coords, "coords")
        idx, dist, ws = knn_forward_raw(coords, row_splits, K, direction, tf_compat)
        order = cell_order(ws, coords.shape[0], coords.shape[1], row_splits.numel(), K).clone()
        ctx.save_for_backward(idx, coords, order)
        ctx.mark_non_differentiable(idx, order)
        # no zero tensors for the gradients of idx and order (an int64 [N, K] fill per backward)
        ctx.set_materialize_grads(False)
        return idx, dist, order

    @staticmethod
    def backward(ctx, grad_idx, grad_dist, grad_order):
        idx, coords, order = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None, None, None, None
        if grad_dist is None:
            return torch.zeros_like(coords), None, None, None, None
        return (knn_backward_raw(grad_dist.to(dtype=torch.float32).contiguous(), idx, coords, order),
                None, None, None, None)


def binned_select_knn_with_order(K: int, coords: torch.Tensor, row_splits: torch.Tensor,
                                 direction: Optional[torch.Tensor] = None,
                                 n_bins: Optional[torch.Tensor] = None, max_bin_dims: int = 3,
                                 torch_compatible_indices: bool = False
                                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """binned_select_knn that also returns the cell order of its search grid: (idx, distsq,
    order) with order int32 [N], a permutation of the points that keeps spatial neighbours
    together.  Kernels that walk the neighbour rows (GravNet aggregation) use it as their
    processing order for cache locality.

    Written in the TorchScript subset (the reference's wrapper is ``@torch.jit.script``,
    extensions/binned_select_knn.py:11): modules that call it can be scripted, traced, saved and
    loaded; the work happens in the dispatcher op ``fgc_b200::knn_forward``."""
    if coords.dim() != 2:
        raise ValueError("coords must be [N, D]")
    if coords.shape[1] == 0:
        raise ValueError("Input coordinates must have at least one dimension. Got 0 dimensions.")
    if max_bin_dims <= 0:
        raise ValueError("max_bin_dims must be greater than 0. Got 0.")
    if coords.shape[1] < 2:
        # the reference supports 2..5 binning dimensions only (binned_select_knn_cpu.cpp:278)
        raise ValueError("Unsupported number of binning dimensions.")
    if coords.shape[1] > 16:
        raise ValueError("Unsupported number of coordinate dimensions (2..16).")
    if K < 1 or K > 257:
        raise ValueError("binned_select_knn: K must be in 1..257")
    if coords.dtype != torch.float32:
        coords = coords.to(dtype=torch.float32)
    if n_bins is not None:
        if not bool((n_bins > 0).all()):
            raise RuntimeError("BinByCoordinates: n_bins must be greater than zero.")
    coords = coords.contiguous()
    row_splits = row_splits.to(device=coords.device, dtype=torch.int64).contiguous()
    dirn: Optional[torch.Tensor] = None
    if direction is not None:
        if direction.numel() > 0:
            if direction.numel() != coords.shape[0]:
                raise ValueError("direction must have one entry per point")
            dirn = direction.detach().to(device=coords.device, dtype=torch.int64).contiguous()
    if torch.jit.is_scripting():
        idx, dist, order = torch.ops.fgc_b200.knn_forward(coords, row_splits, K, dirn, torch_compatible_indices)
        return idx, dist, order
    else:
        if torch.jit.is_tracing() or torch.compiler.is_compiling():
            return torch.ops.fgc_b200.knn_forward(coords, row_splits, K, dirn, torch_compatible_indices)
        return _BinnedKNN.apply(coords, row_splits, K, dirn, torch_compatible_indices)


def binned_select_knn(K: int, coords: torch.Tensor, row_splits: torch.Tensor,
                      direction: Optional[torch.Tensor] = None,
                      n_bins: Optional[torch.Tensor] = None, max_bin_dims: int = 3,
                      torch_compatible_indices: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """K nearest neighbours inside each row split.

    Args:
        K: number of neighbours including the point itself.
        coords: [N, D] coordinates, 2 <= D <= 16 (converted to float32).
        row_splits: ragged-tensor row splits; neighbours never cross a split.
        direction: optional [N] tensor; 0: can only be a neighbour, 1: can only have
            neighbours, 2: neither.
        n_bins, max_bin_dims: accepted for compatibility and validated like the
            reference does.  They tune the reference's internal binning and do not
            change which points are nearest; this implementation sizes its own
            search grid from the data.
        torch_compatible_indices: fill unused slots with the point's own index instead of -1.

    Returns:
        (indices int64 [N,K], squared distances float32 [N,K]).  Slot 0 is the point
        itself; the order of the other slots is unspecified, as in the reference (it is
        the same on every run, though).  Differentiable w.r.t. coords through the distances.
    """
    if not torch.jit.is_scripting():
        # conveniences outside TorchScript: python numbers / lists where the reference takes tensors
        if not isinstance(row_splits, torch.Tensor):
            row_splits = torch.tensor(row_splits, dtype=torch.int64, device=coords.device)
        if n_bins is not None and not isinstance(n_bins, torch.Tensor):
            n_bins = torch.tensor(n_bins, dtype=torch.int64)
    idx, dist, order = binned_select_knn_with_order(K, coords, row_splits, direction, n_bins, max_bin_dims,
                                                    torch_compatible_indices)
    return idx, dist
