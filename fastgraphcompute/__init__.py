"""``fastgraphcompute`` -- the reference's import path, served by the sm_100a implementation.

Code written against FastGraphCompute imports ``fastgraphcompute``, ``fastgraphcompute.extensions.*``,
``fastgraphcompute.gnn_ops`` and ``fastgraphcompute.torch_geometric_interface``
(fastgraphcompute/__init__.py:5-8 and extensions/__init__.py:2-13 of the reference).  With this
directory on the path those imports resolve to the modules of ``fastgraphcompute_b200``: the
names below are aliases, not copies, so there is one implementation and one set of module-level
switches.  The reference's dispatcher op names (``torch.ops.fastgraphcompute_custom_ops.*``,
``torch.ops.bin_by_coordinates.*``, ``torch.ops.binned_select_knn.*``,
``torch.ops.binned_select_knn_grad.*``, ``torch.ops.index_replacer.*``) are published too, unless
the reference's own op library is already loaded in this process.

CUDA tensors only, like the package it points to.
"""
import importlib
import sys

import fastgraphcompute_b200 as _impl
from fastgraphcompute_b200 import (bin_by_coordinates, binned_select_knn, index_replacer,  # noqa: F401
                                   oc_helper_matrices, select_with_default)

__version__ = "1.0.1"      # the interface version this package stands in for (setup.cfg:3 of the reference)

_ALIASES = (
    "extensions",
    "extensions.bin_by_coordinates",
    "extensions.binned_select_knn",
    "extensions.index_replacer",
    "extensions.oc_helper",
    "gnn_ops",
    "torch_geometric_interface",
)
for _name in _ALIASES:
    _mod = importlib.import_module("fastgraphcompute_b200." + _name)
    sys.modules[__name__ + "." + _name] = _mod
    if "." not in _name:
        globals()[_name] = _mod

_impl.torch_ops.register_reference_op_names()

__all__ = ["bin_by_coordinates", "binned_select_knn", "index_replacer", "oc_helper_matrices",
           "select_with_default"]
