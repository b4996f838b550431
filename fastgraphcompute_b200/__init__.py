"""fastgraphcompute_b200 -- sm_100a implementation of FastGraphCompute's spatial-graph
hot path behind the reference's Python entry points (fastgraphcompute/__init__.py:5-8).

    from fastgraphcompute_b200 import bin_by_coordinates, binned_select_knn, index_replacer
    from fastgraphcompute_b200.gnn_ops import GravNetOp

CUDA tensors only; the CUDA library libfgc_b200.so must have been built
(python fastgraphcompute_b200/build.py).
"""
from . import torch_ops  # noqa: F401  (registers the fgc_b200 dispatcher ops)
from .extensions.bin_by_coordinates import bin_by_coordinates
from .extensions.binned_select_knn import binned_select_knn
from .extensions.index_replacer import index_replacer
from .extensions.oc_helper import oc_helper_matrices, select_with_default
from .extensions.select_knn import select_knn

__version__ = "0.1.0"
__all__ = ["bin_by_coordinates", "binned_select_knn", "index_replacer", "select_with_default",
           "oc_helper_matrices", "select_knn"]
