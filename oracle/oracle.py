"""TEST INFRASTRUCTURE ONLY: numpy front of the C oracle (oracle/fgc_oracle.c).

Mirrors the call signatures of the reference's Python entry points so that the
parity tests read like the reference's own tests; everything works on numpy
arrays on the CPU.  Only tests, the smoke check and the CPU-baseline leg of the
benchmark may import this module.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libfgc_oracle.so")
        if not os.path.exists(path):
            from . import build_oracle
            build_oracle.build()
        _LIB = ctypes.CDLL(path)
        _LIB.oracle_default_n_bins.restype = ctypes.c_int64
    return _LIB


def _f(a):
    return a.ctypes.data_as(_f32p)


def _i(a):
    return a.ctypes.data_as(_i64p) if a is not None else None


def _c64(x):
    return ctypes.c_int64(int(x))


def bin_by_coordinates(coordinates, row_splits, bin_width=None, n_bins=None,
                       calc_n_per_bin=True, pre_normalized=False):
    """Oracle for bin_by_coordinates (extensions/bin_by_coordinates.py:11-111).

    Returns (bin_indices[N,D+1] i64, flat[N] i64, n_bins[D] i64, bin_width[1] f32, n_per_bin i64).
    Raises ValueError for the input errors the reference rejects.
    """
    L = _lib()
    coords = np.array(coordinates, dtype=np.float32, order="C", copy=True)
    N, D = coords.shape
    rs = np.ascontiguousarray(row_splits, dtype=np.int64)
    bw = np.zeros(1, np.float32)
    nb = np.zeros(D, np.int64)
    have_bw = bin_width is not None
    have_nb = n_bins is not None
    if have_bw:
        bw[0] = np.asarray(bin_width, np.float32).reshape(-1)[0]
    if have_nb:
        nbv = np.asarray(n_bins, np.int64).reshape(-1)
        nb[:] = nbv[0] if nbv.size == 1 else nbv
    rc = L.oracle_bin_prepare(_f(coords), _c64(N), _c64(D), int(pre_normalized), int(have_bw),
                              _f(bw), int(have_nb), _i(nb))
    if rc:
        raise ValueError({1: "BinByCoordinates: input coordinates contain non-finite values",
                          2: "BinByCoordinates: dmax_coords must be greater than zero.",
                          3: "Either bin_width or n_bins must be provided.",
                          4: "BinByCoordinates: n_bins must be greater than zero.",
                          5: "BinByCoordinates: bin_width must be greater than zero."}[rc])
    n_total = int(np.prod(nb)) * (len(rs) - 1)
    assigned = np.zeros((N, D + 1), np.int64)
    flat = np.zeros(N, np.int64)
    nper = np.zeros(n_total, np.int64)
    L.oracle_bin_assign(_f(coords), _i(rs), ctypes.c_float(bw[0]), _i(nb), _i(assigned), _i(flat),
                        _i(nper), _c64(N), _c64(D), _c64(len(rs)), _c64(n_total),
                        int(calc_n_per_bin))
    return assigned, flat, nb, bw, nper


def default_n_bins(row_splits, K, max_bin_dims):
    rs = np.ascontiguousarray(row_splits, dtype=np.int64)
    return int(_lib().oracle_default_n_bins(_i(rs), _c64(len(rs)), _c64(K), _c64(max_bin_dims)))


def binned_select_knn(K, coords, row_splits, direction=None, n_bins=None, max_bin_dims=3,
                      torch_compatible_indices=False, return_evals=False):
    """Oracle for binned_select_knn forward (extensions/binned_select_knn.py:12-94).

    Returns (idx[N,K] i64, distsq[N,K] f32) in the reference's slot order
    (slot 0 = self, then visiting/replacement order, -1 pads last).
    """
    L = _lib()
    c = np.ascontiguousarray(coords, dtype=np.float32)
    N, D = c.shape
    if D == 0:
        raise ValueError("Input coordinates must have at least one dimension. Got 0 dimensions.")
    if max_bin_dims == 0:
        raise ValueError("max_bin_dims must be greater than 0. Got 0.")
    mbd = max(min(int(max_bin_dims), D, 5), 2)
    rs = np.ascontiguousarray(row_splits, dtype=np.int64)
    dirn = None if direction is None else np.ascontiguousarray(direction, dtype=np.int64)
    nb = None if n_bins is None else np.ascontiguousarray(np.asarray(n_bins, np.int64).reshape(-1))
    idx = np.zeros((N, K), np.int64)
    dist = np.zeros((N, K), np.float32)
    evals = ctypes.c_int64(0)
    rc = L.oracle_binned_select_knn(_f(c), _c64(N), _c64(D), _i(rs), _c64(len(rs)), _c64(K),
                                    _i(dirn), _i(nb), _c64(0 if nb is None else nb.size),
                                    _c64(mbd), int(torch_compatible_indices), _i(idx), _f(dist),
                                    ctypes.byref(evals))
    if rc == 20:
        raise ValueError("Unsupported number of binning dimensions.")
    if rc:
        raise ValueError("oracle binning error %d" % rc)
    if return_evals:
        return idx, dist, evals.value
    return idx, dist


def binned_select_knn_grad(grad_distsq, idx, coords):
    """Oracle for the kNN backward (binned_select_knn_grad_cpu.cpp:96-164)."""
    L = _lib()
    g = np.ascontiguousarray(grad_distsq, dtype=np.float32)
    ix = np.ascontiguousarray(idx, dtype=np.int64)
    c = np.ascontiguousarray(coords, dtype=np.float32)
    N, D = c.shape
    out = np.zeros((N, D), np.float32)
    L.oracle_knn_grad(_f(g), _i(ix), _f(c), _f(out), _c64(N), _c64(ix.shape[1]), _c64(D))
    return out


def index_replacer(to_be_replaced, replacements):
    """Oracle for index_replacer (index_replacer_cpu.cpp:7-26)."""
    L = _lib()
    t = np.ascontiguousarray(to_be_replaced, dtype=np.int64)
    r = np.ascontiguousarray(replacements, dtype=np.int64)
    out = np.empty_like(t)
    L.oracle_index_replacer(_i(t), _i(r), _i(out), _c64(t.size), _c64(r.shape[0]))
    return out


def select_with_default(idx, feat, default_value):
    """Oracle for select_with_default (extensions/oc_helper.py:232-271)."""
    idx = np.asarray(idx, np.int64)
    feat = np.asarray(feat)
    out = np.full(idx.shape + (feat.shape[1],), default_value, dtype=feat.dtype)
    valid = idx != -1
    out[valid] = feat[idx[valid]]
    return out


def select_knn(K, coords, row_splits, max_radius=-1.0):
    """Oracle for the reference's brute-force op select_knn::select_knn (select_knn.cpp:60-62,
    select_knn_cpu.cpp:9-206): (idx [N,K] i64, distsq [N,K] f32); max_radius <= 0: no radius."""
    L = _lib()
    c = np.ascontiguousarray(coords, dtype=np.float32)
    rs = np.ascontiguousarray(row_splits, dtype=np.int64)
    N, D = c.shape
    idx = np.zeros((N, K), np.int64)
    dist = np.zeros((N, K), np.float32)
    r2 = np.float32(float(max_radius) * float(max_radius)) if max_radius > 0 else np.float32(max_radius)
    L.oracle_select_knn(_f(c), _i(rs), _c64(len(rs)), _c64(N), _c64(K), _c64(D), ctypes.c_float(float(r2)),
                        _i(idx), _f(dist))
    return idx, dist


def oc_helper_matrices(truth_idxs, row_splits, calc_m_not=True):
    """Oracle for oc_helper_matrices (extensions/oc_helper.py:128-230): the unique
    (truth index, row split) pairs with a non-negative index (oc_helper.py:100-118), the two
    scalar sizes (oc_helper_helper.cpp:31-93) and the per-object scans of calc_m
    (oc_helper_cpu.cpp:14-83).  Objects are listed by (row split, truth index) -- what a stable
    argsort gives at oc_helper.py:187; the reference's own order there is unspecified, so
    callers compare the rows as a set keyed by their first entry.

    Returns (M [K, n_maxuq], M_not [K, n_maxrs], objects_per_split [R])."""
    asso = np.asarray(truth_idxs, np.int64).reshape(-1)
    rs = np.asarray(row_splits, np.int64)
    n_splits = len(rs) - 1
    objects = []
    per_split = np.zeros(n_splits, np.int64)
    n_maxuq = 0
    for e in range(n_splits):
        part = asso[rs[e]:rs[e + 1]]
        vals = np.unique(part[part >= 0])
        per_split[e] = len(vals)
        for v in vals:
            objects.append((e, int(v)))
            n_maxuq = max(n_maxuq, int((part == v).sum()))
    n_maxrs = int((rs[1:] - rs[:-1]).max()) if n_splits > 0 else 0
    M = np.full((len(objects), n_maxuq), -1, np.int64)
    M_not = np.full((len(objects), n_maxrs), -1, np.int64)
    for k, (e, v) in enumerate(objects):
        fill = fill_not = 0
        for i_v in range(int(rs[e]), int(rs[e + 1])):
            if asso[i_v] == v:
                M[k, fill] = i_v
                fill += 1
            elif calc_m_not:
                M_not[k, fill_not] = i_v
                fill_not += 1
    return M, M_not, per_split


def gravnet_aggregate_fwd(prop, idx, distsq):
    """Oracle for steps 4-7 of GravNetOp.forward (gnn_ops.py:90-102)."""
    L = _lib()
    p = np.ascontiguousarray(prop, dtype=np.float32)
    ix = np.ascontiguousarray(idx, dtype=np.int64)
    d = np.ascontiguousarray(distsq, dtype=np.float32)
    N, P = p.shape
    K = ix.shape[1]
    mean = np.zeros((N, P), np.float32)
    mx = np.zeros((N, P), np.float32)
    am = np.zeros((N, P), np.int32)
    L.oracle_gravnet_fwd(_f(p), _i(ix), _f(d), _c64(N), _c64(K), _c64(P), _f(mean), _f(mx),
                         am.ctypes.data_as(_i32p))
    return mean, mx, am


def gravnet_aggregate_bwd(prop, idx, distsq, argmax, g_mean, g_max):
    """Oracle for the backward of the aggregation (autograd of gnn_ops.py:90-102)."""
    L = _lib()
    p = np.ascontiguousarray(prop, dtype=np.float32)
    ix = np.ascontiguousarray(idx, dtype=np.int64)
    d = np.ascontiguousarray(distsq, dtype=np.float32)
    am = np.ascontiguousarray(argmax, dtype=np.int32)
    gm = np.ascontiguousarray(g_mean, dtype=np.float32)
    gx = np.ascontiguousarray(g_max, dtype=np.float32)
    N, P = p.shape
    K = ix.shape[1]
    dp = np.zeros((N, P), np.float32)
    dd = np.zeros((N, K), np.float32)
    L.oracle_gravnet_bwd(_f(p), _i(ix), _f(d), am.ctypes.data_as(_i32p), _f(gm), _f(gx), _c64(N),
                         _c64(K), _c64(P), _f(dp), _f(dd))
    return dp, dd
