"""Counterpart of the reference's brute-force op ``select_knn::select_knn`` (select_knn.cpp:60-62;
CPU kernel select_knn_cpu.cpp:74-136, CUDA kernel select_knn_cuda_kernel.cu:73-132), which the
reference ships without a Python wrapper: k nearest neighbours inside row splits with an optional
``max_radius``.

Here it is the grid search of binned_select_knn (which scans a small row split exhaustively
anyway) followed by a radius cut of its result; differentiable through the distances like
binned_select_knn.
"""
from typing import Optional, Tuple

import torch

from .. import _cabi
from .binned_select_knn import binned_select_knn


def select_knn(K: int, coords: torch.Tensor, row_splits: torch.Tensor,
               mask: Optional[torch.Tensor] = None, max_radius: float = -1.0,
               mask_mode: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(idx [N, K] int64, distsq [N, K] float32): slot 0 the point itself, then the nearest
    other points of its row split that lie within ``max_radius`` (<= 0: no radius), -1 pads.

    ``mask`` / ``mask_mode`` are accepted for signature compatibility; the reference's kernels
    never read them."""
    idx, distsq = binned_select_knn(K, coords, row_splits)
    if not max_radius > 0:
        return idx, distsq
    keep = distsq.detach() <= float(torch.tensor(float(max_radius) * float(max_radius), dtype=torch.float32))
    out_idx = idx.clone()
    out_d = distsq.detach().clone()
    with torch.cuda.device(out_idx.device):
        _cabi.check(_cabi.lib.fgc_knn_radius_filter(_cabi.ptr(out_idx), _cabi.ptr(out_d), out_idx.shape[0], K,
                                                    float(max_radius), 0, _cabi.current_stream(out_idx.device)),
                    "fgc_knn_radius_filter")
    if not distsq.requires_grad:
        return out_idx, out_d
    # the same cut through autograd: kept slots keep their gradient path, in the filter's order
    valid = keep & (idx >= 0)
    valid[:, 0] = True
    order = torch.argsort((~valid).to(torch.int8), dim=1, stable=True)
    gathered = torch.gather(torch.where(valid, distsq, torch.zeros_like(distsq)), 1, order)
    return out_idx, gathered
