"""GravNetOp -- drop-in for fastgraphcompute.gnn_ops.GravNetOp (gnn_ops.py:8-109).

Same constructor, sub-module names (so state_dicts are interchangeable) and
returned tuple.  The three Linear layers stay torch (cuBLAS); neighbour search
and the weighted mean/max aggregation with their backward passes run in
libfgc_b200.so.
"""
from typing import Optional, Tuple

import torch

from . import torch_ops  # noqa: F401  (registers the fgc_b200 dispatcher ops)
from .extensions.binned_select_knn import binned_select_knn_with_order


class _GravNetAggregate(torch.autograd.Function):
    """Eager-mode autograd node of the aggregation (fgc_b200::gravnet_aggregate is its
    dispatcher twin for TorchScript and tracing)."""

    @staticmethod
    def forward(ctx, propagate, neighbor_idx, distsq, order):
        fmean, fmax, argmax = torch_ops.gravnet_aggregate_eager(propagate, neighbor_idx, distsq, order)
        ctx.save_for_backward(propagate, neighbor_idx, distsq, argmax)
        ctx.order = order
        ctx.set_materialize_grads(False)
        return fmean, fmax

    @staticmethod
    def backward(ctx, g_mean, g_max):
        prop, idx, dsq, argmax = ctx.saved_tensors
        if g_mean is None:
            g_mean = torch.zeros_like(prop, dtype=torch.float32)
        if g_max is None:
            g_max = torch.zeros_like(prop, dtype=torch.float32)
        d_prop, d_dsq = torch_ops.gravnet_aggregate_backward_eager(prop, idx, dsq, argmax, g_mean, g_max, ctx.order)
        return d_prop, None, d_dsq, None


def gravnet_aggregate(propagate: torch.Tensor, neighbor_idx: torch.Tensor, distsq: torch.Tensor,
                      order: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(mean, max) over the K neighbour slots of exp(-10*distsq)-weighted neighbour features
    (gnn_ops.py:90-102 of the reference, fused; differentiable w.r.t. propagate and distsq).

    order: optional int32 [N] permutation used as processing order (cache locality only)."""
    if torch.jit.is_scripting():
        fmean, fmax, _ = torch.ops.fgc_b200.gravnet_aggregate(propagate, neighbor_idx, distsq, order)
        return fmean, fmax
    else:
        if torch.jit.is_tracing() or torch.compiler.is_compiling():
            # graph capture (jit.trace, torch.compile) goes through the dispatcher op, which has
            # shape inference and autograd registered; the eager node below talks to the
            # library directly
            fmean, fmax, _ = torch.ops.fgc_b200.gravnet_aggregate(propagate, neighbor_idx, distsq, order)
            return fmean, fmax
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
