"""Mirror of fastgraphcompute.extensions for the spatial-graph hot path."""
from .bin_by_coordinates import bin_by_coordinates
from .binned_select_knn import binned_select_knn
from .index_replacer import index_replacer
from .oc_helper import select_with_default

__all__ = ["bin_by_coordinates", "binned_select_knn", "index_replacer", "select_with_default"]
