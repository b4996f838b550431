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


class _GravNetAggregateCat(torch.autograd.Function):
    """Eager-mode autograd node of the aggregation that writes into [x | mean | max]
    (fgc_b200::gravnet_aggregate_cat is its dispatcher twin)."""

    @staticmethod
    def forward(ctx, x, propagate, neighbor_idx, distsq, order):
        cat, argmax = torch_ops.gravnet_aggregate_cat_eager(x, propagate, neighbor_idx, distsq, order)
        ctx.save_for_backward(propagate, neighbor_idx, distsq, argmax)
        ctx.order = order
        ctx.n_in = x.shape[1]
        ctx.set_materialize_grads(False)
        return cat

    @staticmethod
    def backward(ctx, g_cat):
        if g_cat is None:
            return None, None, None, None, None
        prop, idx, dsq, argmax = ctx.saved_tensors
        g_cat = g_cat.contiguous()
        d_prop, d_dsq = torch_ops.gravnet_aggregate_cat_backward_eager(prop, idx, dsq, argmax, g_cat, ctx.order)
        return (g_cat[:, :ctx.n_in] if ctx.needs_input_grad[0] else None), d_prop, None, d_dsq, None


def gravnet_aggregate_cat(x: torch.Tensor, propagate: torch.Tensor, neighbor_idx: torch.Tensor,
                          distsq: torch.Tensor, order: Optional[torch.Tensor] = None) -> torch.Tensor:
    """cat([x, mean, max], dim=1) of a GravNet layer (gnn_ops.py:90-106 of the reference) with the
    aggregation kernel writing mean and max straight into their columns, and a backward that
    reads the gradient's columns in place.  Differentiable w.r.t. x, propagate and distsq."""
    if torch.jit.is_scripting():
        cat, _ = torch.ops.fgc_b200.gravnet_aggregate_cat(x, propagate, neighbor_idx, distsq, order)
        return cat
    else:
        if torch.jit.is_tracing() or torch.compiler.is_compiling():
            cat, _ = torch.ops.fgc_b200.gravnet_aggregate_cat(x, propagate, neighbor_idx, distsq, order)
            return cat
        return _GravNetAggregateCat.apply(x, propagate, neighbor_idx, distsq, order)


class _GravNetProject(torch.autograd.Function):
    """Eager-mode autograd node of the fused input projections (fgc_b200::gravnet_project is its
    dispatcher twin)."""

    @staticmethod
    def forward(ctx, x, w_space, b_space, w_prop, b_prop):
        space, prop = torch_ops.gravnet_project_eager(x, w_space, b_space, w_prop, b_prop)
        ctx.save_for_backward(x, w_space, w_prop)
        ctx.has_bias = (b_space is not None, b_prop is not None)
        ctx.set_materialize_grads(False)
        return space, prop

    @staticmethod
    def backward(ctx, d_space, d_prop):
        x, w_space, w_prop = ctx.saved_tensors
        need_dx = ctx.needs_input_grad[0]
        dx, dws, dbs, dwp, dbp = torch_ops.gravnet_project_backward_eager(x, w_space, w_prop, d_space, d_prop, need_dx)
        return (dx if need_dx else None, dws, dbs if ctx.has_bias[0] else None, dwp,
                dbp if ctx.has_bias[1] else None)


class _GravNetProjectCat(torch.autograd.Function):
    """Eager-mode node: the fused input projections that also start the matrix [x | mean | max]
    (x written into its first columns by the same pass).  Its backward takes the gradient of that
    matrix and adds its x columns to dx inside the kernel."""

    @staticmethod
    def forward(ctx, x, w_space, b_space, w_prop, b_prop, cat_extra):
        space, prop, cat = torch_ops.gravnet_project_eager(x, w_space, b_space, w_prop, b_prop, cat_extra)
        ctx.save_for_backward(x, w_space, w_prop)
        ctx.has_bias = (b_space is not None, b_prop is not None)
        ctx.set_materialize_grads(False)
        return space, prop, cat

    @staticmethod
    def backward(ctx, d_space, d_prop, d_cat):
        x, w_space, w_prop = ctx.saved_tensors
        need_dx = ctx.needs_input_grad[0]
        dx, dws, dbs, dwp, dbp = torch_ops.gravnet_project_backward_eager(x, w_space, w_prop, d_space, d_prop,
                                                                          need_dx, d_cat)
        return (dx if need_dx else None, dws, dbs if ctx.has_bias[0] else None, dwp,
                dbp if ctx.has_bias[1] else None, None)


class _GravNetAggregateInto(torch.autograd.Function):
    """Eager-mode node: the aggregation writing mean and max into their columns of the matrix that
    _GravNetProjectCat started (in place).  The gradient of the matrix passes through to that node,
    which reads only its x columns; this node reads the mean and max columns."""

    @staticmethod
    def forward(ctx, cat, propagate, neighbor_idx, distsq, order, n_in):
        argmax = torch_ops.gravnet_aggregate_into_eager(cat, n_in, propagate, neighbor_idx, distsq, order)
        ctx.mark_dirty(cat)
        ctx.save_for_backward(propagate, neighbor_idx, distsq, argmax)
        ctx.order = order
        ctx.set_materialize_grads(False)
        return cat

    @staticmethod
    def backward(ctx, g_cat):
        if g_cat is None:
            return None, None, None, None, None, None
        prop, idx, dsq, argmax = ctx.saved_tensors
        g_cat = g_cat.contiguous()
        d_prop, d_dsq = torch_ops.gravnet_aggregate_cat_backward_eager(prop, idx, dsq, argmax, g_cat, ctx.order)
        return g_cat, d_prop, None, d_dsq, None, None


def gravnet_project_and_aggregate(x: torch.Tensor, w_space: torch.Tensor, b_space: Optional[torch.Tensor],
                                  w_prop: torch.Tensor, b_prop: Optional[torch.Tensor], k: int,
                                  row_splits: torch.Tensor
                                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Everything of a GravNet layer in front of its output transformation (gnn_ops.py:79-106 of the
    reference): (cat([x, mean, max], 1), neighbor_idx, distsq, space).

    In eager mode x is copied into the matrix by the projection kernel, mean and max are written
    into it by the aggregation kernel, and the two gradients of x (through the matrix and through the
    projections) are added inside the projection backward.  Under TorchScript, tracing and
    torch.compile the same result comes from the dispatcher ops."""
    if torch.jit.is_scripting():
        space, prop = torch.ops.fgc_b200.gravnet_project(x, w_space, b_space, w_prop, b_prop)
        neighbor_idx, distsq, order = binned_select_knn_with_order(k, space.contiguous(), row_splits)
        cat, _ = torch.ops.fgc_b200.gravnet_aggregate_cat(x, prop, neighbor_idx, distsq, order)
        return cat, neighbor_idx, distsq, space
    else:
        if torch.jit.is_tracing() or torch.compiler.is_compiling() or not x.is_cuda:
            space, prop = gravnet_project(x, w_space, b_space, w_prop, b_prop)
            neighbor_idx, distsq, order = binned_select_knn_with_order(k, space.contiguous(), row_splits)
            return gravnet_aggregate_cat(x, prop, neighbor_idx, distsq, order), neighbor_idx, distsq, space
        x = x.to(torch.float32)
        space, prop, cat = _GravNetProjectCat.apply(x, w_space, b_space, w_prop, b_prop, 2 * w_prop.shape[0])
        neighbor_idx, distsq, order = binned_select_knn_with_order(k, space.contiguous(), row_splits)
        cat = _GravNetAggregateInto.apply(cat, prop, neighbor_idx, distsq, order, x.shape[1])
        return cat, neighbor_idx, distsq, space


def gravnet_project(x: torch.Tensor, w_space: torch.Tensor, b_space: Optional[torch.Tensor],
                    w_prop: torch.Tensor, b_prop: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """The two input projections of a GravNet layer, (x @ w_space^T + b_space, x @ w_prop^T + b_prop)
    (gnn_ops.py:79-82 of the reference), computed in one pass over x, with a fused backward that
    reads x and the two output gradients once.  Differentiable w.r.t. all five arguments."""
    if torch.jit.is_scripting():
        space, prop = torch.ops.fgc_b200.gravnet_project(x, w_space, b_space, w_prop, b_prop)
        return space, prop
    else:
        if torch.jit.is_tracing() or torch.compiler.is_compiling():
            space, prop = torch.ops.fgc_b200.gravnet_project(x, w_space, b_space, w_prop, b_prop)
            return space, prop
        return _GravNetProject.apply(x, w_space, b_space, w_prop, b_prop)


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
        # both projections in one pass over x, [x | mean | max] without a concatenation pass; the
        # parameters stay in the Linear modules (state_dict as in the reference)
        cat, neighbor_idx, distsq, space = gravnet_project_and_aggregate(
            x, self.space_transformations.weight, self.space_transformations.bias,
            self.propagate_transformations.weight, self.propagate_transformations.bias, self.k, row_splits)
        out = self.output_transformations(cat)
        return out, neighbor_idx, distsq, space
