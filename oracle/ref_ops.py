"""TEST INFRASTRUCTURE ONLY: thin access to the reference's own CPU ops.

Loads oracle/_ref/binned_knn_ops.so (built by oracle/build_ref.py from the
reference's unmodified .cpp files) and calls its dispatcher ops directly:

  bin_by_coordinates::bin_by_coordinates           (bin_by_coordinates.cpp:143-153)
  fastgraphcompute_custom_ops::binned_select_knn_autograd
                                                   (binned_knn_autograd_kernel.cpp:271-277)
  index_replacer::index_replacer                   (index_replacer.cpp:43-53)

The argument normalisation that the reference performs in Python before these
calls (extensions/binned_select_knn.py:36-92, extensions/bin_by_coordinates.py:
33-109) is restated here so that no reference Python file has to be imported.
Only tests, the smoke check and the CPU-baseline leg of the benchmark may use
this module; the product never does.
"""
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "binned_knn_ops.so")
_loaded = False


def available():
    return os.path.exists(_SO)


def load():
    global _loaded
    if not _loaded:
        if not available():
            raise RuntimeError("oracle/_ref/binned_knn_ops.so missing: run python oracle/build_ref.py")
        torch.ops.load_library(_SO)
        _loaded = True


def ref_bin_by_coordinates(coordinates, row_splits, bin_width=None, n_bins=None,
                           calc_n_per_bin=True, pre_normalized=False):
    """Reference bin_by_coordinates on CPU tensors (extensions/bin_by_coordinates.py:11-111)."""
    load()
    coords = coordinates.clone()
    if not torch.isfinite(coords).all():
        raise ValueError("BinByCoordinates: input coordinates contain non-finite values")
    if not pre_normalized:
        coords = coords - torch.min(coords, dim=0, keepdim=True).values
    dmax = torch.max(coords, dim=0).values
    dmin = torch.min(coords, dim=0).values
    dmax = torch.where(dmin == dmax, dmax + 1.0, dmax)
    dmax = dmax + 1e-3
    dmax = torch.where(torch.isfinite(dmax), dmax, torch.ones_like(dmax))
    if bin_width is None:
        if n_bins is None:
            raise ValueError("Either bin_width or n_bins must be provided.")
        if not torch.is_tensor(n_bins):
            n_bins = torch.tensor(n_bins, dtype=torch.int64)
        if n_bins.dim() == 0:
            n_bins = n_bins.repeat(coords.shape[1])
        bin_width = torch.max(dmax / n_bins.to(torch.float32)).unsqueeze(-1)
    elif n_bins is None:
        n_bins = (dmax / bin_width).to(torch.int64) + 1
    return torch.ops.bin_by_coordinates.bin_by_coordinates(
        coords, row_splits.to(torch.int64), bin_width, n_bins, calc_n_per_bin, pre_normalized)


def ref_binned_select_knn(K, coords, row_splits, direction=None, n_bins=None,
                          max_bin_dims=3, torch_compatible_indices=False):
    """Reference binned_select_knn on CPU tensors (extensions/binned_select_knn.py:12-94).

    Differentiable w.r.t. coords through the returned distsq, exactly as the
    reference (BinnedKNNAutograd, binned_knn_autograd_kernel.cpp:84-253).
    """
    load()
    if coords.shape[1] == 0:
        raise ValueError("Input coordinates must have at least one dimension. Got 0 dimensions.")
    if max_bin_dims == 0:
        raise ValueError("max_bin_dims must be greater than 0. Got 0.")
    max_bin_dims = max(min(int(max_bin_dims), coords.shape[1], 5), 2)
    if coords.dtype != torch.float32:
        coords = coords.to(torch.float32)
    if n_bins is not None and not torch.is_tensor(n_bins):
        n_bins = torch.tensor(n_bins, dtype=torch.int64)
    coords = coords.clone().contiguous() if coords.requires_grad else coords.contiguous()
    row_splits = row_splits.contiguous().to(torch.int64)
    if direction is not None:
        direction = direction.contiguous()
    if n_bins is not None:
        n_bins = n_bins.contiguous().to(torch.int64)
    return torch.ops.fastgraphcompute_custom_ops.binned_select_knn_autograd(
        coords, row_splits, int(K), direction, n_bins, max_bin_dims, bool(torch_compatible_indices))


def ref_index_replacer(to_be_replaced, replacements):
    """Reference index_replacer (extensions/index_replacer.py:40-59)."""
    load()
    return torch.ops.index_replacer.index_replacer(to_be_replaced, replacements)


def ref_select_with_default(idx, feat, default_value):
    """Restatement of select_with_default (extensions/oc_helper.py:232-271)."""
    idx = idx.long()
    V, K = idx.shape
    F = feat.shape[1]
    out = torch.full((V, K, F), default_value, dtype=feat.dtype, device=feat.device)
    valid = idx != -1
    pos = valid.nonzero()
    out[pos[:, 0], pos[:, 1]] = feat[idx[valid]]
    return out


def ref_gravnet_aggregate(propagate, neighbor_idx, distsq):
    """Steps 4-7 of GravNetOp.forward (gnn_ops.py:90-102) in plain torch (autograd-capable)."""
    weights = torch.exp(-10. * distsq)
    g = ref_select_with_default(neighbor_idx, propagate, 0.0)
    g = g * weights.unsqueeze(-1)
    return torch.mean(g, dim=1), torch.max(g, dim=1).values


class RefGravNetOp(torch.nn.Module):
    """GravNetOp of the reference (gnn_ops.py:40-109) with the reference CPU kNN underneath.

    Same sub-module names, so a state_dict moves freely between this class, the
    reference's own class and the B200 module.
    """

    def __init__(self, in_channels, out_channels, space_dimensions, propagate_dimensions, k,
                 output_activation=None):
        super().__init__()
        self.k = k
        self.space_transformations = torch.nn.Linear(in_channels, space_dimensions)
        self.propagate_transformations = torch.nn.Linear(in_channels, propagate_dimensions)
        self.output_transformations = torch.nn.Sequential(
            torch.nn.Linear(in_channels + 2 * propagate_dimensions, out_channels),
            output_activation if output_activation is not None else torch.nn.ReLU())

    def forward(self, x, row_splits):
        space = self.space_transformations(x)
        propagate = self.propagate_transformations(x)
        idx, distsq = ref_binned_select_knn(self.k, space.contiguous(), row_splits)
        fmean, fmax = ref_gravnet_aggregate(propagate, idx, distsq)
        out = self.output_transformations(torch.cat([x, fmean, fmax], dim=1))
        return out, idx, distsq, space


# --------------------------------------------------------------------------- oc_helper

_OC_SOS = [os.path.join(_HERE, "_ref", "oc_helper_cpu.so"), os.path.join(_HERE, "_ref", "oc_helper_helper.so")]
_oc_loaded = False


def oc_available():
    return all(os.path.exists(p) for p in _OC_SOS)


def ref_oc_helper_matrices(truth_idxs, row_splits, calc_m_not=True):
    """Reference oc_helper_matrices on CPU tensors: the orchestration of
    extensions/oc_helper.py:100-230 restated around the reference's own ops
    oc_helper_helper::max_same_valued_entries_per_row_split (oc_helper_helper.cpp:31-93) and
    oc_helper_cpu::oc_helper_cpu (oc_helper_cpu.cpp:117-156).  The argsort that orders the
    objects by row split is made stable here (the reference's is not, so its order among the
    objects of one row split is unspecified)."""
    global _oc_loaded
    if not _oc_loaded:
        if not oc_available():
            raise RuntimeError("oracle/_ref/oc_helper_*.so missing: run python oracle/build_ref.py")
        for p in _OC_SOS:
            torch.ops.load_library(p)
        _oc_loaded = True
    truth_idxs = truth_idxs.to(torch.int64)
    row_splits = row_splits.to(torch.int64)
    lengths = row_splits[1:] - row_splits[:-1]
    max_length = torch.max(lengths)
    row_ids = torch.repeat_interleave(torch.arange(len(lengths), dtype=torch.int64), lengths)
    pairs = torch.stack((truth_idxs, row_ids), dim=1)
    pairs = torch.unique(pairs[pairs[:, 0] != -1], dim=0)
    pairs = pairs[pairs[:, 0] >= 0]
    _, max_same, per_split = torch.ops.oc_helper_helper.max_same_valued_entries_per_row_split(
        truth_idxs, row_splits, True)
    order = torch.argsort(pairs[:, 1], stable=True)
    unique_idxs = pairs[order, 0].contiguous()
    unique_rs = pairs[order, 1].contiguous()
    M, M_not = torch.ops.oc_helper_cpu.oc_helper_cpu(
        truth_idxs.contiguous(), unique_idxs, unique_rs, row_splits.contiguous(),
        max_same.to(torch.int64).reshape(1), max_length.reshape(1), bool(calc_m_not))
    return M, M_not, per_split


# --------------------------------------------------------------------------- brute-force select_knn

_SELECT_SO = os.path.join(_HERE, "_ref", "select_knn_lib.so")
_select_loaded = False


def select_knn_available():
    return os.path.exists(_SELECT_SO)


def ref_select_knn(K, coords, row_splits, max_radius=-1.0):
    """The reference's brute-force op select_knn::select_knn on CPU tensors (select_knn.cpp:60-62
    -> select_knn_cpu.cpp:161-206).  The mask arguments are passed as the op wants them; its CPU
    kernel never reads them."""
    global _select_loaded
    if not _select_loaded:
        if not select_knn_available():
            raise RuntimeError("oracle/_ref/select_knn_lib.so missing: run python oracle/build_ref.py")
        torch.ops.load_library(_SELECT_SO)
        _select_loaded = True
    mask = torch.zeros(coords.shape[0], dtype=torch.int64)
    return torch.ops.select_knn.select_knn(coords.to(torch.float32).contiguous(), row_splits.to(torch.int64).contiguous(),
                                           mask, int(K), float(max_radius), 0)
