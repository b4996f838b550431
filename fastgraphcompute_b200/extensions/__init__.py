"""Mirror of fastgraphcompute.extensions (extensions/__init__.py:2-13 of the reference)."""
from .bin_by_coordinates import bin_by_coordinates
from .binned_select_knn import binned_select_knn
from .index_replacer import index_replacer
from .oc_helper import oc_helper_matrices, select_with_default

__all__ = ["bin_by_coordinates", "binned_select_knn", "index_replacer", "oc_helper_matrices",
           "select_with_default"]
