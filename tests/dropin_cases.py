"""Checks of the ``fastgraphcompute`` import path, run in a process of its own by
test_gpu_dropin.py (the alias publishes the reference's dispatcher op names, which must not
meet the reference's own op library in one process).  Prints DROPIN-OK when everything held."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import fastgraphcompute                                             # noqa: E402
import fastgraphcompute.extensions                                  # noqa: E402
from fastgraphcompute import bin_by_coordinates, binned_select_knn, index_replacer  # noqa: E402
from fastgraphcompute.extensions.binned_select_knn import binned_select_knn as knn2  # noqa: E402
from fastgraphcompute.gnn_ops import GravNetOp                      # noqa: E402
from fastgraphcompute.torch_geometric_interface import row_splits_from_strict_batch  # noqa: E402

import fastgraphcompute_b200                                        # noqa: E402
import parity                                                       # noqa: E402
from oracle import oracle                                           # noqa: E402

DEV = "cuda:0"


def main():
    assert knn2 is binned_select_knn is fastgraphcompute_b200.binned_select_knn
    import importlib
    assert importlib.import_module("fastgraphcompute.extensions.binned_select_knn") is \
        sys.modules["fastgraphcompute_b200.extensions.binned_select_knn"]
    assert importlib.import_module("fastgraphcompute.gnn_ops") is sys.modules["fastgraphcompute_b200.gnn_ops"]
    g = torch.Generator().manual_seed(11)
    n, K = 3000, 12
    coords = torch.rand((n, 3), generator=g)
    rs = torch.tensor([0, 1100, 1100, 3000], dtype=torch.int64)
    oidx, odsq = oracle.binned_select_knn(K, coords.numpy(), rs.numpy())

    # 1. the reference's autograd op name
    idx, dsq = torch.ops.fastgraphcompute_custom_ops.binned_select_knn_autograd(
        coords.to(DEV), rs.to(DEV), K, None, None, 3, False)
    parity.assert_knn_parity(idx.cpu().numpy(), dsq.cpu().numpy(), oidx, odsq, what="autograd op name")

    # 2. the low-level search on caller-binned, caller-sorted input, fed the way
    #    BinnedKNNAutograd::forward feeds it (extensions/binned_knn_autograd_kernel.cpp:108-168)
    c = coords.to(DEV)
    n_bins = torch.tensor([6, 6, 6], dtype=torch.int64, device=DEV)
    bin_idx, flat, nb, bw, n_per_bin = torch.ops.bin_by_coordinates.bin_by_coordinates(
        c, rs.to(DEV), None, n_bins, True, False)
    order = torch.argsort(flat)
    s_coords = c.index_select(0, order).contiguous()
    bounds = torch.cat([torch.zeros(1, dtype=torch.int64, device=DEV), torch.cumsum(n_per_bin, 0)])
    s_idx, s_dsq = torch.ops.binned_select_knn.binned_select_knn(
        s_coords, flat.index_select(0, order), bin_idx.index_select(0, order).contiguous(), bounds, nb, bw,
        torch.empty(0, dtype=torch.int64, device=DEV), False, False, K)
    # indices refer to the sorted order; the sorted points are the oracle's input here
    sidx, sdsq = oracle.binned_select_knn(K, s_coords.cpu().numpy(), rs.numpy())
    parity.assert_knn_parity(s_idx.cpu().numpy(), s_dsq.cpu().numpy(), sidx, sdsq, what="low-level op")
    # ... and the reference's next two steps bring them back to the original order
    back = torch.ops.index_replacer.index_replacer(s_idx, order)
    full = torch.empty_like(back)
    full[order] = back
    fd = torch.empty_like(s_dsq)
    fd[order] = s_dsq
    parity.assert_knn_parity(full.cpu().numpy(), fd.cpu().numpy(), oidx, odsq, what="low-level op, unsorted")

    # 3. gradient op name
    gd = torch.randn((n, K), generator=g)
    grad = torch.ops.binned_select_knn_grad.binned_select_knn_grad(gd.to(DEV), idx, dsq, c)
    og = oracle.binned_select_knn_grad(gd.numpy(), idx.cpu().numpy(), coords.numpy())
    parity.assert_grad_close(grad.cpu().numpy(), og, what="gradient op name")

    # 4. module and helpers through the reference's paths
    m = GravNetOp(8, 16, 3, 8, 6).to(DEV)
    out = m(torch.randn((200, 8), device=DEV), torch.tensor([0, 80, 200], dtype=torch.int32, device=DEV))
    assert out[0].shape == (200, 16)
    assert row_splits_from_strict_batch(torch.tensor([0, 0, 1, 1, 1], device=DEV)).tolist() == [0, 2, 5]
    r = index_replacer(torch.tensor([[0, -1, 2]], device=DEV), torch.tensor([5, 6, 7], device=DEV))
    assert r.tolist() == [[5, -1, 7]]
    b = bin_by_coordinates(c, rs.to(DEV), n_bins=torch.tensor(5))
    assert b[0].shape == (n, 4)
    print("DROPIN-OK")


if __name__ == "__main__":
    main()
