"""ctypes binding of libfgc_b200.so (declared in include/fgc_b200.h).

There is no CPU or eager-PyTorch fallback behind these calls: if the library is
missing, importing this module raises, and tensors that are not on a CUDA device
are rejected.
"""
import ctypes
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FGC_B200_LIB") or os.path.join(_PKG_DIR, "libfgc_b200.so")

if not os.path.exists(LIB_PATH):
    raise RuntimeError(
        "fastgraphcompute_b200: %s is missing. Build it with "
        "`python fastgraphcompute_b200/build.py` (needs nvcc; targets sm_100a). "
        "There is no fallback implementation." % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

c_void_p = ctypes.c_void_p
c_i64 = ctypes.c_int64
c_i32 = ctypes.c_int32
c_size = ctypes.c_size_t
c_float = ctypes.c_float

FGC_MAX_BIN_DIMS = 8
FGC_MAX_K = 257

# kernels launched per call (for launch accounting in benchmarks)
KERNELS_BUILD_GRID = 9
KERNELS_BUILD_GRID_D4 = 11      # D = 4: a second density pass may follow a fallback to three binned coordinates
KERNELS_PUBLISH_STATUS = 1   # the wrapper's status check after the grid build
KERNELS_SEARCH = 2             # k_knn + k_knn_hard (the queries that gave up their walk)
KERNELS_KNN_BWD = 1
KERNELS_KNN_BWD_SORTED = 7   # reverse graph (6) + gather (1)
KERNELS_GRAVNET_PROJECT = 2    # forward + backward of the fused input projections
KERNELS_GRAVNET_FWD = 1
KERNELS_GRAVNET_BWD = 1
KERNELS_OC_PREPARE = 8          # + the radix sort's own kernels

STATUS_NONFINITE = 1
STATUS_BAD_ROW_SPLITS = 2
STATUS_BAD_DMAX = 4
STATUS_BAD_NBINS = 8
STATUS_BAD_BINWIDTH = 16
STATUS_INTERNAL = 32

ERR_BAD_ARGUMENT = -1
ERR_UNSUPPORTED_DIM = -2
ERR_UNSUPPORTED_K = -3
ERR_WORKSPACE = -4
ERR_TOO_LARGE = -5
ERR_STATIC_TOO_LARGE = -6
STATIC_WORKSPACE_BYTES = 4 << 20


class BinParams(ctypes.Structure):
    """Host mirror of fgc_bin_params (256 bytes)."""
    _fields_ = [
        ("status", c_i32), ("n_coords", c_i32), ("bin_width", c_float), ("reserved0", c_i32),
        ("shift", c_float * FGC_MAX_BIN_DIMS),
        ("n_bins", c_i64 * FGC_MAX_BIN_DIMS),
        ("scratch", ctypes.c_uint32 * (2 * FGC_MAX_BIN_DIMS + 2)),
        ("pad", ctypes.c_uint8 * 72),
    ]


assert ctypes.sizeof(BinParams) == 256

# name -> (restype, argtypes); the single source for the symbol-export test
SIGNATURES = {
    "fgc_version": (ctypes.c_int, []),
    "fgc_error_string": (ctypes.c_char_p, [ctypes.c_int]),
    "fgc_bin_prepare": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_i32, c_void_p, c_void_p, c_i32,
                                       c_void_p, c_void_p]),
    "fgc_bin_assign": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_void_p, c_i64, c_void_p, c_i32,
                                      c_i64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fgc_knn_workspace_bytes": (c_size, [c_i64, c_i32, c_i64, c_i32]),
    "fgc_binned_knn_fwd": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_void_p, c_i64, c_i32, c_void_p,
                                          c_i32, c_float, c_void_p, c_void_p, c_void_p, c_size,
                                          c_void_p]),
    "fgc_knn_build_grid": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_void_p, c_i64, c_i32, c_void_p,
                                          c_float, c_void_p, c_size, c_void_p]),
    "fgc_knn_build_grid_dims": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_void_p, c_i64, c_i32, c_void_p,
                                               c_float, c_i32, c_void_p, c_size, c_void_p]),
    "fgc_knn_publish_grid_info": (ctypes.c_int, [c_void_p, c_void_p, c_void_p]),
    "fgc_knn_search": (ctypes.c_int, [c_i64, c_i32, c_i64, c_i32, c_i32, c_i32, c_i32, c_void_p,
                                      c_void_p, c_void_p, c_size, c_void_p]),
    "fgc_knn_read_counters": (ctypes.c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint64),
                                             ctypes.POINTER(c_i32), ctypes.POINTER(c_float),
                                             c_void_p]),
    "fgc_binned_knn_fwd_static": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_void_p, c_i64, c_i32,
                                                 c_void_p, c_i32, c_float, c_void_p, c_void_p,
                                                 c_void_p, c_void_p]),
    "fgc_read_status": (ctypes.c_int, [c_void_p, ctypes.POINTER(c_i32), c_void_p]),
    "fgc_publish_status": (ctypes.c_int, [c_void_p, c_void_p, c_void_p]),
    "fgc_binned_knn_bwd": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i32, c_i32,
                                          c_void_p, c_void_p]),
    "fgc_binned_knn_bwd_ordered": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i32, c_i32, c_void_p,
                                                  c_void_p, c_void_p]),
    "fgc_reverse_graph_bytes": (c_size, [c_i64, c_i32]),
    "fgc_build_reverse_graph": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_void_p, c_size, c_void_p]),
    "fgc_binned_knn_bwd_sorted": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i32, c_i32,
                                                 c_void_p, c_size, c_void_p, c_void_p]),
    "fgc_index_replacer": (ctypes.c_int, [c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p]),
    "fgc_gravnet_aggregate_fwd": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i32, c_i32,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fgc_gravnet_aggregate_bwd": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_void_p, c_i64, c_i32, c_i32, c_void_p, c_void_p,
                                                 c_void_p, c_void_p]),
    "fgc_gravnet_aggregate_bwd_sorted": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                        c_void_p, c_i64, c_i32, c_i32, c_void_p, c_size,
                                                        c_void_p, c_void_p, c_void_p, c_void_p]),
    "fgc_gravnet_aggregate_fwd_ld": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i32, c_i32,
                                                    c_void_p, c_void_p, c_i64, c_void_p, c_void_p, c_void_p]),
    "fgc_gravnet_aggregate_bwd_ld": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                    c_void_p, c_i64, c_i64, c_i32, c_i32, c_void_p, c_void_p,
                                                    c_void_p, c_void_p]),
    "fgc_gravnet_aggregate_bwd_sorted_ld": (ctypes.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                           c_void_p, c_i64, c_i64, c_i32, c_i32, c_void_p, c_size,
                                                           c_void_p, c_void_p, c_void_p, c_void_p]),
    "fgc_knn_cell_order": (c_void_p, [c_void_p, c_i64, c_i32, c_i64, c_i32]),
    "fgc_knn_radius_filter": (ctypes.c_int, [c_void_p, c_void_p, c_i64, c_i32, ctypes.c_double, c_i32, c_void_p]),
    "fgc_oc_workspace_bytes": (c_size, [c_i64]),
    "fgc_oc_prepare": (ctypes.c_int, [c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_size, c_void_p, c_void_p]),
    "fgc_oc_read_sizes": (ctypes.c_int, [c_void_p, ctypes.POINTER(c_i32), ctypes.POINTER(c_i64), c_void_p]),
    "fgc_oc_fill": (ctypes.c_int, [c_void_p, c_size, c_i64, c_void_p, c_i64, c_i64, c_i64, c_void_p, c_void_p,
                                   c_void_p]),
    "fgc_select_with_default": (ctypes.c_int, [c_void_p, c_i64, c_void_p, c_i64, c_i64, c_i32, c_void_p,
                                               c_void_p, c_void_p]),
    "fgc_gravnet_project_fwd_cat": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_i32, c_i32, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_void_p]),
    "fgc_gravnet_project_bwd_cat": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_i32, c_i32, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_i64, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p]),
    "fgc_gravnet_project_supported": (ctypes.c_int, [c_i32, c_i32, c_i32]),
    "fgc_gravnet_project_fwd": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_i32, c_i32, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_void_p]),
    "fgc_gravnet_project_bwd": (ctypes.c_int, [c_void_p, c_i64, c_i32, c_i32, c_i32, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p]),
    "fgc_pyg_workspace_bytes": (c_size, [c_i64]),
    "fgc_row_splits_from_strict_batch": (ctypes.c_int, [c_void_p, c_i64, c_void_p, c_void_p, c_size, c_void_p]),
    "fgc_pyg_read_count": (ctypes.c_int, [c_void_p, ctypes.POINTER(c_i64), c_void_p]),
    "fgc_strict_batch_from_row_splits": (ctypes.c_int, [c_void_p, c_i64, c_i64, c_void_p, c_void_p]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def error_string(code):
    return lib.fgc_error_string(int(code)).decode()


def check(code, what):
    """Raise for a non-zero return value of the library."""
    if code == 0:
        return
    msg = "%s failed: %s (code %d)" % (what, error_string(code), code)
    if code in (ERR_UNSUPPORTED_DIM, ERR_UNSUPPORTED_K, ERR_BAD_ARGUMENT):
        raise ValueError(msg)
    raise RuntimeError(msg)


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


def require_cuda(t, name):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor" % name)
    if not t.is_cuda:
        raise RuntimeError(
            "fastgraphcompute_b200 runs on CUDA tensors only (no CPU fallback): %s is on %s"
            % (name, t.device))


def current_stream(device):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)
