"""Dispatcher registration of the hot-path ops (namespace ``fgc_b200``).

The reference exposes its native code as dispatcher ops (``TORCH_LIBRARY`` blocks in
extensions/binned_knn_autograd_kernel.cpp:271-277, bin_by_coordinates.cpp:143-153,
binned_select_knn_grad.cpp:58-69, index_replacer.cpp:43-53), which is what makes its Python
wrappers and ``GravNetOp`` usable from TorchScript (script / trace / save / load).  The ops
below do the same for this implementation: each one unpacks tensors into device pointers and
calls the C ABI of libfgc_b200.so; autograd is attached with ``register_autograd`` and shape
inference with ``register_fake``.

    torch.ops.fgc_b200.knn_forward(coords, row_splits, K, direction, tf_compat) -> (idx, distsq, order)
    torch.ops.fgc_b200.knn_backward(grad_distsq, idx, coords, order) -> grad_coords
    torch.ops.fgc_b200.gravnet_aggregate(prop, idx, distsq, order) -> (mean, max, argmax)
    torch.ops.fgc_b200.gravnet_aggregate_backward(...) -> (d_prop, d_distsq)
    torch.ops.fgc_b200.index_replacer(to_be_replaced, replacements) -> replaced
    torch.ops.fgc_b200.bin_by_coordinates(...) -> (bin_indices, flat, n_bins, bin_width, n_per_bin)

``register_reference_op_names()`` additionally publishes them under the reference's own op
names, for scripted code that calls ``torch.ops.<reference namespace>.*`` directly.
"""
import ctypes
import importlib
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _cabi

_knn = importlib.import_module(__package__ + ".extensions.binned_select_knn")

# GravNet aggregation backward by sorted-segment gathers over the reverse neighbour graph instead
# of float atomics (P <= 128, N*K < 2^31): bit-identical gradients from run to run, about 3x the
# time of the atomic kernel.  Together with binned_select_knn.deterministic_backward a whole
# GravNetOp training step becomes reproducible.
deterministic_gravnet_backward = False


# --------------------------------------------------------------------------- kNN

@torch.library.custom_op("fgc_b200::knn_forward", mutates_args=())
def knn_forward(coords: Tensor, row_splits: Tensor, K: int, direction: Optional[Tensor],
                tf_compat: bool) -> Tuple[Tensor, Tensor, Tensor]:
    _cabi.require_cuda(coords, "coords")
    coords = coords.to(torch.float32).contiguous()
    row_splits = row_splits.to(device=coords.device, dtype=torch.int64).contiguous()
    if direction is not None:
        direction = direction.to(device=coords.device, dtype=torch.int64).contiguous()
    idx, dist, ws = _knn.knn_forward_raw(coords, row_splits, int(K), direction, bool(tf_compat))
    order = _knn.cell_order(ws, coords.shape[0], coords.shape[1], row_splits.numel(), int(K)).clone()
    return idx, dist, order


@knn_forward.register_fake
def _(coords, row_splits, K, direction, tf_compat):
    n = coords.shape[0]
    return (coords.new_empty((n, K), dtype=torch.int64), coords.new_empty((n, K), dtype=torch.float32),
            coords.new_empty((n,), dtype=torch.int32))


@torch.library.custom_op("fgc_b200::knn_backward", mutates_args=())
def knn_backward(grad_distsq: Tensor, idx: Tensor, coords: Tensor, order: Optional[Tensor]) -> Tensor:
    _cabi.require_cuda(coords, "coords")
    grad_distsq = grad_distsq.to(torch.float32).contiguous()
    idx = idx.to(torch.int64).contiguous()
    coords = coords.to(torch.float32).contiguous()
    if order is not None:
        order = order.to(torch.int32).contiguous()
    return _knn.knn_backward_raw(grad_distsq, idx, coords, order)


@knn_backward.register_fake
def _(grad_distsq, idx, coords, order):
    return torch.empty_like(coords, dtype=torch.float32)


def _knn_setup(ctx, inputs, output):
    coords = inputs[0]
    idx = output[0]
    ctx.save_for_backward(idx, coords, output[2])


def _knn_grad(ctx, g_idx, g_dist, g_order):
    idx, coords, order = ctx.saved_tensors
    if g_dist is None:
        return torch.zeros_like(coords), None, None, None, None
    return torch.ops.fgc_b200.knn_backward(g_dist, idx, coords.to(torch.float32), order), None, None, None, None


knn_forward.register_autograd(_knn_grad, setup_context=_knn_setup)


# --------------------------------------------------------------------------- GravNet aggregation

def gravnet_aggregate_eager(prop: Tensor, idx: Tensor, distsq: Tensor,
                            order: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    """(mean, max, argmax) straight from the library (no dispatcher round trip)."""
    _cabi.require_cuda(prop, "propagate")
    prop = prop.to(torch.float32).contiguous()
    idx = idx.to(torch.int64).contiguous()
    distsq = distsq.to(torch.float32).contiguous()
    if order is not None:
        order = order.to(torch.int32).contiguous()
    n_vert, P = prop.shape
    K = idx.shape[1]
    fmean = torch.empty((n_vert, P), dtype=torch.float32, device=prop.device)
    fmax = torch.empty_like(fmean)
    argmax = torch.empty((n_vert, P), dtype=torch.int32, device=prop.device)
    with torch.cuda.device(prop.device):
        _cabi.check(_cabi.lib.fgc_gravnet_aggregate_fwd(
            _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), n_vert, K, P, _cabi.ptr(fmean),
            _cabi.ptr(fmax), _cabi.ptr(argmax), _cabi.ptr(order),
            _cabi.current_stream(prop.device)), "fgc_gravnet_aggregate_fwd")
    return fmean, fmax, argmax


@torch.library.custom_op("fgc_b200::gravnet_aggregate", mutates_args=())
def gravnet_aggregate(prop: Tensor, idx: Tensor, distsq: Tensor,
                      order: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    return gravnet_aggregate_eager(prop, idx, distsq, order)


@gravnet_aggregate.register_fake
def _(prop, idx, distsq, order):
    return (torch.empty_like(prop, dtype=torch.float32), torch.empty_like(prop, dtype=torch.float32),
            torch.empty_like(prop, dtype=torch.int32))


def gravnet_aggregate_backward_eager(prop: Tensor, idx: Tensor, distsq: Tensor, argmax: Tensor,
                                     g_mean: Tensor, g_max: Tensor,
                                     order: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    """(d_prop, d_distsq) straight from the library."""
    prop = prop.to(torch.float32).contiguous()
    idx = idx.to(torch.int64).contiguous()
    distsq = distsq.to(torch.float32).contiguous()
    g_mean = g_mean.to(torch.float32).contiguous()
    g_max = g_max.to(torch.float32).contiguous()
    n_vert, P = prop.shape
    K = idx.shape[1]
    d_prop = torch.empty_like(prop)
    d_dsq = torch.empty_like(distsq)
    argmax = argmax.contiguous()
    with torch.cuda.device(prop.device):
        stream = _cabi.current_stream(prop.device)
        rg, rbytes = None, 0
        if deterministic_gravnet_backward and P <= 128:
            # kept for the kNN backward of the same layer, which scatters through the same indices
            rg, rbytes = _knn.reverse_graph(idx, keep=_knn.deterministic_backward)
        if rbytes:
            _cabi.check(_cabi.lib.fgc_gravnet_aggregate_bwd_sorted(
                _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), _cabi.ptr(argmax), _cabi.ptr(g_mean),
                _cabi.ptr(g_max), n_vert, K, P, _cabi.ptr(rg), rbytes, _cabi.ptr(d_prop), _cabi.ptr(d_dsq),
                _cabi.ptr(order), stream), "fgc_gravnet_aggregate_bwd_sorted")
        else:
            _cabi.check(_cabi.lib.fgc_gravnet_aggregate_bwd(
                _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), _cabi.ptr(argmax),
                _cabi.ptr(g_mean), _cabi.ptr(g_max), n_vert, K, P, _cabi.ptr(d_prop), _cabi.ptr(d_dsq),
                _cabi.ptr(order), stream), "fgc_gravnet_aggregate_bwd")
    return d_prop, d_dsq


@torch.library.custom_op("fgc_b200::gravnet_aggregate_backward", mutates_args=())
def gravnet_aggregate_backward(prop: Tensor, idx: Tensor, distsq: Tensor, argmax: Tensor,
                               g_mean: Tensor, g_max: Tensor,
                               order: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return gravnet_aggregate_backward_eager(prop, idx, distsq, argmax, g_mean, g_max, order)


@gravnet_aggregate_backward.register_fake
def _(prop, idx, distsq, argmax, g_mean, g_max, order):
    return torch.empty_like(prop, dtype=torch.float32), torch.empty_like(distsq, dtype=torch.float32)


def _agg_setup(ctx, inputs, output):
    prop, idx, distsq, order = inputs
    ctx.save_for_backward(prop, idx, distsq, output[2])
    ctx.order = order


def _agg_grad(ctx, g_mean, g_max, g_argmax):
    prop, idx, distsq, argmax = ctx.saved_tensors
    if g_mean is None:
        g_mean = torch.zeros_like(prop, dtype=torch.float32)
    if g_max is None:
        g_max = torch.zeros_like(prop, dtype=torch.float32)
    d_prop, d_dsq = torch.ops.fgc_b200.gravnet_aggregate_backward(prop, idx, distsq, argmax, g_mean,
                                                                   g_max, ctx.order)
    return d_prop, None, d_dsq, None


gravnet_aggregate.register_autograd(_agg_grad, setup_context=_agg_setup)


# ------------------------------------------------------- aggregation written into [x | mean | max]

def gravnet_aggregate_cat_eager(x: Tensor, prop: Tensor, idx: Tensor, distsq: Tensor,
                                order: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    """(cat, argmax): cat = [x | mean | max] as one [N, C + 2P] matrix, the aggregation kernel
    writing its two results straight into their columns (gnn_ops.py:90-106 of the reference
    without the separate concatenation pass)."""
    _cabi.require_cuda(prop, "propagate")
    prop = prop.to(torch.float32).contiguous()
    idx = idx.to(torch.int64).contiguous()
    distsq = distsq.to(torch.float32).contiguous()
    if order is not None:
        order = order.to(torch.int32).contiguous()
    n_vert, P = prop.shape
    C = x.shape[1]
    K = idx.shape[1]
    cat = torch.empty((n_vert, C + 2 * P), dtype=torch.float32, device=prop.device)
    cat[:, :C].copy_(x)
    argmax = torch.empty((n_vert, P), dtype=torch.int32, device=prop.device)
    with torch.cuda.device(prop.device):
        _cabi.check(_cabi.lib.fgc_gravnet_aggregate_fwd_ld(
            _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), n_vert, K, P, _cabi.ptr(cat[:, C:C + P]),
            _cabi.ptr(cat[:, C + P:]), C + 2 * P, _cabi.ptr(argmax), _cabi.ptr(order),
            _cabi.current_stream(prop.device)), "fgc_gravnet_aggregate_fwd_ld")
    return cat, argmax


def gravnet_aggregate_into_eager(cat: Tensor, n_in: int, prop: Tensor, idx: Tensor, distsq: Tensor,
                                 order: Optional[Tensor]) -> Tensor:
    """Writes mean and max into columns n_in.. of cat ([N, n_in + 2P], row-major) in place and
    returns the argmax tensor."""
    _cabi.require_cuda(prop, "propagate")
    prop = prop.to(torch.float32).contiguous()
    idx = idx.to(torch.int64).contiguous()
    distsq = distsq.to(torch.float32).contiguous()
    if order is not None:
        order = order.to(torch.int32).contiguous()
    n_vert, P = prop.shape
    K = idx.shape[1]
    if (cat.dtype != torch.float32 or cat.dim() != 2 or cat.shape[0] != n_vert or cat.shape[1] != n_in + 2 * P
            or not cat.is_contiguous()):
        raise ValueError("gravnet_aggregate_into: cat must be a contiguous float32 [N, n_in + 2P] matrix")
    argmax = torch.empty((n_vert, P), dtype=torch.int32, device=prop.device)
    with torch.cuda.device(prop.device):
        _cabi.check(_cabi.lib.fgc_gravnet_aggregate_fwd_ld(
            _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), n_vert, K, P, _cabi.ptr(cat[:, n_in:n_in + P]),
            _cabi.ptr(cat[:, n_in + P:]), n_in + 2 * P, _cabi.ptr(argmax), _cabi.ptr(order),
            _cabi.current_stream(prop.device)), "fgc_gravnet_aggregate_fwd_ld")
    return argmax


@torch.library.custom_op("fgc_b200::gravnet_aggregate_cat", mutates_args=())
def gravnet_aggregate_cat(x: Tensor, prop: Tensor, idx: Tensor, distsq: Tensor,
                          order: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return gravnet_aggregate_cat_eager(x, prop, idx, distsq, order)


@gravnet_aggregate_cat.register_fake
def _(x, prop, idx, distsq, order):
    return (x.new_empty((x.shape[0], x.shape[1] + 2 * prop.shape[1]), dtype=torch.float32),
            torch.empty_like(prop, dtype=torch.int32))


def gravnet_aggregate_cat_backward_eager(prop: Tensor, idx: Tensor, distsq: Tensor, argmax: Tensor,
                                         g_cat: Tensor, order: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    """(d_prop, d_distsq) from the gradient of [x | mean | max]: the kernels read the mean and
    max columns in place (row stride C + 2P), no slices are copied."""
    prop = prop.to(torch.float32).contiguous()
    idx = idx.to(torch.int64).contiguous()
    distsq = distsq.to(torch.float32).contiguous()
    g_cat = g_cat.to(torch.float32).contiguous()
    n_vert, P = prop.shape
    K = idx.shape[1]
    ld = g_cat.shape[1]
    C = ld - 2 * P
    g_mean, g_max = g_cat[:, C:C + P], g_cat[:, C + P:]
    d_prop = torch.empty_like(prop)
    d_dsq = torch.empty_like(distsq)
    argmax = argmax.contiguous()
    with torch.cuda.device(prop.device):
        stream = _cabi.current_stream(prop.device)
        rg, rbytes = None, 0
        if deterministic_gravnet_backward and P <= 128:
            rg, rbytes = _knn.reverse_graph(idx, keep=_knn.deterministic_backward)
        if rbytes:
            _cabi.check(_cabi.lib.fgc_gravnet_aggregate_bwd_sorted_ld(
                _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), _cabi.ptr(argmax), _cabi.ptr(g_mean),
                _cabi.ptr(g_max), ld, n_vert, K, P, _cabi.ptr(rg), rbytes, _cabi.ptr(d_prop), _cabi.ptr(d_dsq),
                _cabi.ptr(order), stream), "fgc_gravnet_aggregate_bwd_sorted_ld")
        else:
            _cabi.check(_cabi.lib.fgc_gravnet_aggregate_bwd_ld(
                _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(distsq), _cabi.ptr(argmax),
                _cabi.ptr(g_mean), _cabi.ptr(g_max), ld, n_vert, K, P, _cabi.ptr(d_prop), _cabi.ptr(d_dsq),
                _cabi.ptr(order), stream), "fgc_gravnet_aggregate_bwd_ld")
    return d_prop, d_dsq


@torch.library.custom_op("fgc_b200::gravnet_aggregate_cat_backward", mutates_args=())
def gravnet_aggregate_cat_backward(prop: Tensor, idx: Tensor, distsq: Tensor, argmax: Tensor,
                                   g_cat: Tensor, order: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return gravnet_aggregate_cat_backward_eager(prop, idx, distsq, argmax, g_cat, order)


@gravnet_aggregate_cat_backward.register_fake
def _(prop, idx, distsq, argmax, g_cat, order):
    return torch.empty_like(prop, dtype=torch.float32), torch.empty_like(distsq, dtype=torch.float32)


def _agg_cat_setup(ctx, inputs, output):
    x, prop, idx, distsq, order = inputs
    ctx.save_for_backward(prop, idx, distsq, output[1])
    ctx.order = order
    ctx.n_in = x.shape[1]


def _agg_cat_grad(ctx, g_cat, g_argmax):
    prop, idx, distsq, argmax = ctx.saved_tensors
    if g_cat is None:
        return None, None, None, None, None
    d_prop, d_dsq = torch.ops.fgc_b200.gravnet_aggregate_cat_backward(prop, idx, distsq, argmax, g_cat,
                                                                       ctx.order)
    return g_cat[:, :ctx.n_in], d_prop, None, d_dsq, None


gravnet_aggregate_cat.register_autograd(_agg_cat_grad, setup_context=_agg_cat_setup)


# --------------------------------------------------------------------------- GravNet input projections

def _project_fused_ok(x: Tensor, w_space: Tensor, w_prop: Tensor) -> bool:
    return bool(x.is_cuda and x.dim() == 2 and x.dtype == torch.float32 and w_space.dtype == torch.float32
                and w_prop.dtype == torch.float32
                and _cabi.lib.fgc_gravnet_project_supported(x.shape[1], w_space.shape[0], w_prop.shape[0]))


def gravnet_project_eager(x: Tensor, w_space: Tensor, b_space: Optional[Tensor], w_prop: Tensor,
                          b_prop: Optional[Tensor], cat_extra: int = 0):
    """(space, propagate) = (x @ w_space^T + b_space, x @ w_prop^T + b_prop) in one pass over x; shapes
    the fused kernel does not take go to the library GEMMs.

    cat_extra > 0: also returns a [N, C + cat_extra] matrix whose first C columns hold x (written by
    the same pass; the other columns are left for the aggregation to fill)."""
    n, C = x.shape
    cat = None
    if cat_extra > 0:
        cat = torch.empty((n, C + cat_extra), dtype=torch.float32, device=x.device)
    if not _project_fused_ok(x, w_space, w_prop):
        if cat is not None:
            cat[:, :C].copy_(x)
            return (torch.nn.functional.linear(x, w_space, b_space), torch.nn.functional.linear(x, w_prop, b_prop),
                    cat)
        return (torch.nn.functional.linear(x, w_space, b_space), torch.nn.functional.linear(x, w_prop, b_prop))
    x = x.contiguous()
    w_space = w_space.contiguous()
    w_prop = w_prop.contiguous()
    S, P = w_space.shape[0], w_prop.shape[0]
    space = torch.empty((n, S), dtype=torch.float32, device=x.device)
    prop = torch.empty((n, P), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.lib.fgc_gravnet_project_fwd_cat(
            _cabi.ptr(x), n, C, S, P, _cabi.ptr(w_space), _cabi.ptr(None if b_space is None else b_space.contiguous()),
            _cabi.ptr(w_prop), _cabi.ptr(None if b_prop is None else b_prop.contiguous()), _cabi.ptr(space),
            _cabi.ptr(prop), _cabi.ptr(cat), C + cat_extra, _cabi.current_stream(x.device)),
            "fgc_gravnet_project_fwd_cat")
    if cat is not None:
        return space, prop, cat
    return space, prop


def gravnet_project_backward_eager(x: Tensor, w_space: Tensor, w_prop: Tensor, d_space: Optional[Tensor],
                                   d_prop: Optional[Tensor], need_dx: bool, d_cat: Optional[Tensor] = None
                                   ) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(dx, dw_space, db_space, dw_prop, db_prop); dx is an empty tensor when need_dx is false.

    d_cat (optional, [N, >= C], row-major): its first C columns are a second gradient of x and are
    added to dx by the kernel that writes it."""
    n, C = x.shape
    S, P = w_space.shape[0], w_prop.shape[0]
    # (the fused kernel adds the CTAs' shares of the weight gradients with float atomics: with the
    # reproducible backward passes switched on, the library GEMMs take over)
    if not _project_fused_ok(x, w_space, w_prop) or deterministic_gravnet_backward:
        ds = d_space if d_space is not None else x.new_zeros((n, S))
        dp = d_prop if d_prop is not None else x.new_zeros((n, P))
        dx = ds @ w_space + dp @ w_prop if need_dx else x.new_empty((0,))
        if need_dx and d_cat is not None:
            dx = dx + d_cat[:, :C]
        return dx, ds.t() @ x, ds.sum(0), dp.t() @ x, dp.sum(0)
    x = x.contiguous()
    ds = None if d_space is None else d_space.to(torch.float32).contiguous()
    dp = None if d_prop is None else d_prop.to(torch.float32).contiguous()
    if d_cat is not None and need_dx:
        d_cat = d_cat.to(torch.float32)
        if d_cat.stride(1) != 1:
            d_cat = d_cat.contiguous()
    else:
        d_cat = None
    dx = torch.empty_like(x) if need_dx else x.new_empty((0,))
    dws = torch.empty_like(w_space, memory_format=torch.contiguous_format)
    dwp = torch.empty_like(w_prop, memory_format=torch.contiguous_format)
    dbs = torch.empty((S,), dtype=torch.float32, device=x.device)
    dbp = torch.empty((P,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.lib.fgc_gravnet_project_bwd_cat(
            _cabi.ptr(x), n, C, S, P, _cabi.ptr(w_space.contiguous()), _cabi.ptr(w_prop.contiguous()), _cabi.ptr(ds),
            _cabi.ptr(dp), _cabi.ptr(d_cat), 0 if d_cat is None else d_cat.stride(0),
            _cabi.ptr(dx) if need_dx else None, _cabi.ptr(dws), _cabi.ptr(dbs), _cabi.ptr(dwp),
            _cabi.ptr(dbp), _cabi.current_stream(x.device)), "fgc_gravnet_project_bwd_cat")
    return dx, dws, dbs, dwp, dbp


@torch.library.custom_op("fgc_b200::gravnet_project", mutates_args=())
def gravnet_project(x: Tensor, w_space: Tensor, b_space: Optional[Tensor], w_prop: Tensor,
                    b_prop: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    return gravnet_project_eager(x, w_space, b_space, w_prop, b_prop)


@gravnet_project.register_fake
def _(x, w_space, b_space, w_prop, b_prop):
    return (x.new_empty((x.shape[0], w_space.shape[0])), x.new_empty((x.shape[0], w_prop.shape[0])))


@torch.library.custom_op("fgc_b200::gravnet_project_backward", mutates_args=())
def gravnet_project_backward(x: Tensor, w_space: Tensor, w_prop: Tensor, d_space: Optional[Tensor],
                             d_prop: Optional[Tensor], need_dx: bool
                             ) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    return gravnet_project_backward_eager(x, w_space, w_prop, d_space, d_prop, need_dx)


@gravnet_project_backward.register_fake
def _(x, w_space, w_prop, d_space, d_prop, need_dx):
    return (torch.empty_like(x) if need_dx else x.new_empty((0,)), torch.empty_like(w_space),
            w_space.new_empty((w_space.shape[0],)), torch.empty_like(w_prop), w_prop.new_empty((w_prop.shape[0],)))


def _project_setup(ctx, inputs, output):
    x, w_space, b_space, w_prop, b_prop = inputs
    ctx.save_for_backward(x, w_space, w_prop)
    ctx.has_bias = (b_space is not None, b_prop is not None)


def _project_grad(ctx, d_space, d_prop):
    x, w_space, w_prop = ctx.saved_tensors
    dx, dws, dbs, dwp, dbp = torch.ops.fgc_b200.gravnet_project_backward(x, w_space, w_prop, d_space, d_prop,
                                                                         ctx.needs_input_grad[0])
    return (dx if ctx.needs_input_grad[0] else None, dws, dbs if ctx.has_bias[0] else None, dwp,
            dbp if ctx.has_bias[1] else None)


gravnet_project.register_autograd(_project_grad, setup_context=_project_setup)


# --------------------------------------------------------------------------- index_replacer, binning

@torch.library.custom_op("fgc_b200::index_replacer", mutates_args=())
def index_replacer(to_be_replaced: Tensor, replacements: Tensor) -> Tensor:
    from .extensions.index_replacer import index_replacer_eager
    return index_replacer_eager(to_be_replaced, replacements)


@index_replacer.register_fake
def _(to_be_replaced, replacements):
    return torch.empty_like(to_be_replaced)


@torch.library.custom_op("fgc_b200::bin_by_coordinates", mutates_args=())
def bin_by_coordinates(coordinates: Tensor, row_splits: Tensor, bin_width: Optional[Tensor],
                       n_bins: Optional[Tensor], calc_n_per_bin: bool,
                       pre_normalized: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    from .extensions.bin_by_coordinates import bin_by_coordinates_impl
    return bin_by_coordinates_impl(coordinates, row_splits, bin_width, n_bins, calc_n_per_bin,
                                   pre_normalized, "")


# no fake implementation: the size of n_per_bin depends on the data


# --------------------------------------------------------------------------- reference op names

_REFERENCE_LIBS = []


def reference_ops_loaded() -> bool:
    """True when some other library (the reference's binned_knn_ops.so) has already defined the
    reference's op names in this process."""
    try:
        torch.ops.fastgraphcompute_custom_ops.binned_select_knn_autograd
        return not _REFERENCE_LIBS
    except (AttributeError, RuntimeError):
        return False


def register_reference_op_names():
    """Publish the ops under the names the reference registers, so that scripted code written
    against ``torch.ops.fastgraphcompute_custom_ops.binned_select_knn_autograd``,
    ``torch.ops.bin_by_coordinates.bin_by_coordinates``,
    ``torch.ops.binned_select_knn.binned_select_knn`` (the search on caller-binned input),
    ``torch.ops.binned_select_knn_grad.binned_select_knn_grad`` and
    ``torch.ops.index_replacer.index_replacer`` resolves to this implementation.  Call it
    instead of loading the reference's binned_knn_ops.so (both in one process would define the
    same schemas twice; when that library is already loaded nothing is registered).  Returns the
    list of namespaces it registered."""
    if _REFERENCE_LIBS:
        return [l.ns for l in _REFERENCE_LIBS]
    if reference_ops_loaded():
        return []

    def knn_autograd(coords, row_splits, K, direction, n_bins, max_bin_dims, torch_compatible_indices):
        idx, dist, _ = torch.ops.fgc_b200.knn_forward(coords, row_splits, K, direction,
                                                      torch_compatible_indices)
        return idx, dist

    def knn_grad(grad_distances, indices, distances, coordinates):
        return torch.ops.fgc_b200.knn_backward(grad_distances, indices, coordinates, None)

    def knn_on_binned_input(coordinates, bin_idx, dim_bin_idx, bin_boundaries, n_bins, bin_width, direction,
                            tf_compat, use_direction, K):
        # The reference's low-level search (extensions/binned_select_knn.cpp:82-91) takes points
        # that the caller has already binned and sorted by bin, and answers with indices into
        # that sorted order.  The caller's bins say where its row splits are (every row split
        # owns prod(n_bins) consecutive bins) and nothing else matters for the result, so the
        # search runs on this library's own grid inside those row splits.
        per_split = int(torch.prod(n_bins.to(torch.int64)).item())
        n_b = bin_boundaries.shape[0] - 1
        if per_split < 1 or n_b % per_split != 0:
            raise RuntimeError("binned_select_knn: bin_boundaries do not hold a whole number of row splits")
        row_splits = bin_boundaries.to(torch.int64)[::per_split].contiguous()
        idx, dist, _ = torch.ops.fgc_b200.knn_forward(coordinates, row_splits, K,
                                                      direction if use_direction else None, tf_compat)
        return idx, dist

    specs = [
        ("fastgraphcompute_custom_ops",
         "binned_select_knn_autograd(Tensor coords, Tensor row_splits, int K, Tensor? direction, "
         "Tensor? n_bins, int max_bin_dims, bool torch_compatible_indices) -> (Tensor, Tensor)",
         "binned_select_knn_autograd", knn_autograd, "CompositeImplicitAutograd"),
        ("bin_by_coordinates",
         "bin_by_coordinates(Tensor coordinates, Tensor row_splits, Tensor? bin_width, Tensor? n_bins, "
         "bool calc_n_per_bin, bool pre_normalized) -> (Tensor, Tensor, Tensor, Tensor, Tensor)",
         "bin_by_coordinates", lambda *a: torch.ops.fgc_b200.bin_by_coordinates(*a), "CompositeImplicitAutograd"),
        ("binned_select_knn_grad",
         "binned_select_knn_grad(Tensor grad_distances, Tensor indices, Tensor distances, Tensor coordinates) -> Tensor",
         "binned_select_knn_grad", knn_grad, "CompositeImplicitAutograd"),
        ("binned_select_knn",
         "binned_select_knn(Tensor coordinates, Tensor bin_idx, Tensor dim_bin_idx, Tensor bin_boundaries, "
         "Tensor n_bins, Tensor bin_width, Tensor direction, bool tf_compat, bool use_direction, int K) "
         "-> (Tensor, Tensor)",
         "binned_select_knn", knn_on_binned_input, "CompositeImplicitAutograd"),
        ("index_replacer",
         "index_replacer(Tensor to_be_replaced, Tensor replacements) -> Tensor",
         "index_replacer", lambda a, b: torch.ops.fgc_b200.index_replacer(a, b), "CompositeImplicitAutograd"),
    ]
    for ns, schema, name, fn, key in specs:
        lib = torch.library.Library(ns, "DEF")
        lib.define(schema)
        lib.impl(name, fn, key)
        _REFERENCE_LIBS.append(lib)
    return [l.ns for l in _REFERENCE_LIBS]
