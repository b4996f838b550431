"""GravNetOp -- drop-in for fastgraphcompute.gnn_ops.GravNetOp (gnn_ops.py:8-109).

Same constructor, sub-module names (so state_dicts are interchangeable) and
returned tuple.  The three Linear layers stay torch (cuBLAS); neighbour search
and the weighted mean/max aggregation with their backward passes run in
libfgc_b200.so.
"""
from typing import Tuple

import torch

from . import _cabi
from .extensions.binned_select_knn import binned_select_knn_with_order


class _GravNetAggregate(torch.autograd.Function):
    """exp(-10 d^2)-weighted mean and max over the neighbour slots (gnn_ops.py:90-102)."""

    @staticmethod
    def forward(ctx, propagate, neighbor_idx, distsq, order):
        _cabi.require_cuda(propagate, "propagate")
        if order is not None:
            order = order.to(torch.int32).contiguous()
        prop = propagate.to(torch.float32).contiguous()
        idx = neighbor_idx.to(torch.int64).contiguous()
        dsq = distsq.to(torch.float32).contiguous()
        n_vert, P = prop.shape
        K = idx.shape[1]
        fmean = torch.empty((n_vert, P), dtype=torch.float32, device=prop.device)
        fmax = torch.empty_like(fmean)
        argmax = torch.empty((n_vert, P), dtype=torch.int32, device=prop.device)
        with torch.cuda.device(prop.device):
            _cabi.check(_cabi.lib.fgc_gravnet_aggregate_fwd(
                _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(dsq), n_vert, K, P, _cabi.ptr(fmean),
                _cabi.ptr(fmax), _cabi.ptr(argmax), _cabi.ptr(order),
                _cabi.current_stream(prop.device)), "fgc_gravnet_aggregate_fwd")
        ctx.save_for_backward(prop, idx, dsq, argmax)
        ctx.order = order
        return fmean, fmax

    @staticmethod
    def backward(ctx, g_mean, g_max):
        prop, idx, dsq, argmax = ctx.saved_tensors
        n_vert, P = prop.shape
        K = idx.shape[1]
        g_mean = (torch.zeros_like(prop) if g_mean is None else g_mean.to(torch.float32)).contiguous()
        g_max = (torch.zeros_like(prop) if g_max is None else g_max.to(torch.float32)).contiguous()
        d_prop = torch.empty_like(prop)
        d_dsq = torch.empty_like(dsq)
        with torch.cuda.device(prop.device):
            _cabi.check(_cabi.lib.fgc_gravnet_aggregate_bwd(
                _cabi.ptr(prop), _cabi.ptr(idx), _cabi.ptr(dsq), _cabi.ptr(argmax),
                _cabi.ptr(g_mean), _cabi.ptr(g_max), n_vert, K, P, _cabi.ptr(d_prop),
                _cabi.ptr(d_dsq), _cabi.ptr(ctx.order), _cabi.current_stream(prop.device)),
                "fgc_gravnet_aggregate_bwd")
        return d_prop, None, d_dsq, None


def gravnet_aggregate(propagate, neighbor_idx, distsq, order=None):
    """(mean, max) over the K neighbour slots of exp(-10*distsq)-weighted neighbour features.

    order: optional int32 [N] permutation used as processing order (cache locality only)."""
    return _GravNetAggregate.apply(propagate, neighbor_idx, distsq, order)


class GravNetOp(torch.nn.Module):
    """One GravNet layer [arxiv:1902.07987]: learned coordinates, kNN, distance-weighted
    mean/max message passing, output transformation.

    Args:
        in_channels, out_channels: feature widths.
        space_dimensions: width of the learned coordinate space used for the kNN.
        propagate_dimensions: width of the features exchanged between neighbours.
        k: number of neighbours (including the point itself).
        output_activation: applied after the last Linear (default ReLU).
        optimization_arguments: accepted and ignored, as in the reference.

    forward(x, row_splits) -> (out, neighbor_idx, distsq, space)
    """

    def __init__(self, in_channels, out_channels, space_dimensions, propagate_dimensions, k,
                 output_activation=torch.nn.ReLU(), optimization_arguments: dict = {}):
        super().__init__()
        self.k = k
        self.space_transformations = torch.nn.Linear(in_channels, space_dimensions)
        self.propagate_transformations = torch.nn.Linear(in_channels, propagate_dimensions)
        self.output_transformations = torch.nn.Sequential(
            torch.nn.Linear(in_channels + 2 * propagate_dimensions, out_channels),
            output_activation)
        self.optimization_arguments = optimization_arguments

    def forward(self, x: torch.Tensor, row_splits: torch.Tensor
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        space = self.space_transformations(x)
        propagate = self.propagate_transformations(x)
        neighbor_idx, distsq, order = binned_select_knn_with_order(self.k, space.contiguous(), row_splits)
        fmean, fmax = gravnet_aggregate(propagate, neighbor_idx, distsq, order)
        out = self.output_transformations(torch.cat([x, fmean, fmax], dim=1))
        return out, neighbor_idx, distsq, space
