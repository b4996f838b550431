"""Comparison rules of the parity tests (numpy, CPU).

kNN rows are compared as SETS (the reference's slot order is its visiting order
and carries no meaning): slot 0 must be the point itself, empty slots must come
last, the sorted squared distances must agree within DIST_RTOL, and the index
sets must be identical -- except that two results may disagree on WHICH of
several candidates whose squared distances differ by at most one ulp was kept.
"""
import numpy as np

DIST_RTOL = 1e-6     # squared distances: relative
GRAD_RTOL = 1e-5     # gradients: relative to the gradient's scale (see assert_grad_close)


def _sorted_rows(idx, dist, pad_self):
    """Sort slots 1.. of every row by (empty-last, distance, index)."""
    idx = np.asarray(idx, np.int64)
    dist = np.asarray(dist, np.float64)
    n, k = idx.shape
    rows = np.arange(n)[:, None]
    empty = (idx[:, 1:] < 0) if not pad_self else (idx[:, 1:] == rows)
    key_d = np.where(empty, np.inf, dist[:, 1:])
    key_i = np.where(empty, np.iinfo(np.int64).max, idx[:, 1:])
    order = np.lexsort((key_i, key_d), axis=1)
    return (np.take_along_axis(key_i, order, 1), np.take_along_axis(key_d, order, 1),
            np.take_along_axis(empty, order, 1))


def assert_knn_parity(idx, dist, ref_idx, ref_dist, pad_self=False, what=""):
    """Raise AssertionError unless (idx, dist) matches (ref_idx, ref_dist) under the parity rule.

    Returns a dict of statistics (rows with a tie-substitution, max relative distance error).
    """
    idx = np.asarray(idx, np.int64)
    ref_idx = np.asarray(ref_idx, np.int64)
    dist = np.asarray(dist, np.float32)
    ref_dist = np.asarray(ref_dist, np.float32)
    assert idx.shape == ref_idx.shape and dist.shape == ref_dist.shape, what + " shape mismatch"
    n, k = idx.shape
    if n == 0:
        return dict(rows=0, tie_rows=0, max_rel=0.0)
    assert np.array_equal(idx[:, 0], np.arange(n)), what + " slot 0 must be the point itself"
    assert np.all(dist[:, 0] == 0), what + " slot 0 distance must be 0"
    # empty slots: last in the row, distance 0
    empty = (idx[:, 1:] < 0) if not pad_self else (idx[:, 1:] == np.arange(n)[:, None])
    if k > 1:
        assert np.all(empty[:, 1:] >= empty[:, :-1]), what + " empty slots must be last"
        assert np.all(dist[:, 1:][empty] == 0), what + " empty slots must have distance 0"
    a_i, a_d, a_e = _sorted_rows(idx, dist, pad_self)
    b_i, b_d, b_e = _sorted_rows(ref_idx, ref_dist, pad_self)
    assert np.array_equal(a_e, b_e), what + " number of neighbours per row differs"
    fin = ~a_e
    rel = np.abs(a_d[fin] - b_d[fin]) / np.maximum(np.abs(b_d[fin]), 1e-30)
    rel[(a_d[fin] == b_d[fin])] = 0.0
    max_rel = float(rel.max()) if rel.size else 0.0
    assert max_rel <= DIST_RTOL, "%s distsq differs: max rel err %g" % (what, max_rel)
    bad_rows = np.nonzero((a_i != b_i).any(axis=1))[0]
    tie_rows = 0
    for r in bad_rows:
        mine = dict(zip(a_i[r][~a_e[r]].tolist(), a_d[r][~a_e[r]].tolist()))
        ref = dict(zip(b_i[r][~b_e[r]].tolist(), b_d[r][~b_e[r]].tolist()))
        only_mine = [mine[i] for i in mine if i not in ref]
        only_ref = [ref[i] for i in ref if i not in mine]
        if not only_mine and not only_ref:
            continue   # same set, equal-distance entries in a different order
        assert len(only_mine) == len(only_ref), "%s row %d: set sizes differ" % (what, r)
        d_all = np.array(only_mine + only_ref, np.float32)
        spread = float(d_all.max() - d_all.min())
        assert spread <= float(np.spacing(d_all.max())), (
            "%s row %d: index sets differ beyond a 1-ulp tie (distances %s vs %s)"
            % (what, r, only_mine, only_ref))
        # a substituted candidate must sit at the boundary of the row (the K-th distance)
        kth = np.float32(max(ref.values()))
        assert abs(float(d_all.max()) - float(kth)) <= 2 * float(np.spacing(kth)), (
            "%s row %d: substitution away from the K-th distance" % (what, r))
        tie_rows += 1
    return dict(rows=n, tie_rows=tie_rows, max_rel=max_rel)


def assert_grad_close(a, b, rtol=GRAD_RTOL, what="", scale=None):
    """|a-b| <= rtol * (|b| + scale) elementwise, scale = RMS of b unless given (floating-point
    sums in a different order cannot be compared element-relative where terms cancel; pass the
    magnitude of the summed terms as `scale` for a quantity that is analytically ~0)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    assert a.shape == b.shape, what + " shape mismatch"
    if b.size == 0:
        return 0.0
    if scale is None:
        scale = float(np.sqrt(np.mean(b * b)))
    err = np.abs(a - b) / (np.abs(b) + scale + 1e-30)
    m = float(err.max())
    assert m <= rtol, "%s: max scaled error %g > %g" % (what, m, rtol)
    return m


def brute_force_knn(coords, row_splits, K):
    """Exact fp32 kNN per row split with the reference's distance arithmetic (numpy, O(n^2))."""
    c = np.asarray(coords, np.float32)
    rs = np.asarray(row_splits, np.int64)
    n = c.shape[0]
    idx = np.full((n, K), -1, np.int64)
    dist = np.zeros((n, K), np.float32)
    for e in range(len(rs) - 1):
        lo, hi = int(rs[e]), int(rs[e + 1])
        if hi <= lo:
            continue
        x = c[lo:hi]
        d = np.zeros((hi - lo, hi - lo), np.float32)
        for k in range(c.shape[1]):
            diff = (x[:, None, k] - x[None, :, k]).astype(np.float32)
            d = (d + diff * diff).astype(np.float32)
        np.fill_diagonal(d, -1.0)   # self first
        m = min(K, hi - lo)
        part = np.argsort(d, axis=1, kind="stable")[:, :m]
        idx[lo:hi, :m] = part + lo
        dd = np.take_along_axis(d, part, 1)
        dd[:, 0] = 0
        dist[lo:hi, :m] = dd
    return idx, dist


def canonical_object_rows(M, M_not):
    """Rows of (M, M_not) ordered by the first point of every object.  The order of the objects
    is left open by the reference (oc_helper.py:91-92, its own test sorts too:
    tests/test_oc_helper.py:10-26); the first member id identifies an object uniquely."""
    M = np.asarray(M, np.int64)
    M_not = np.asarray(M_not, np.int64)
    if M.shape[0] == 0:
        return M, M_not
    order = np.argsort(M[:, 0], kind="stable")
    return M[order], M_not[order]


def assert_oc_matrices_equal(M, M_not, per_split, ref_M, ref_M_not, ref_per_split, what=""):
    """Bit-exact equality of the index matrices up to the order of the objects."""
    assert np.array_equal(np.asarray(per_split, np.int64), np.asarray(ref_per_split, np.int64)), what + " objects per split"
    assert tuple(np.shape(M)) == tuple(np.shape(ref_M)), what + " M shape %s vs %s" % (np.shape(M), np.shape(ref_M))
    assert tuple(np.shape(M_not)) == tuple(np.shape(ref_M_not)), what + " M_not shape"
    a, an = canonical_object_rows(M, M_not)
    b, bn = canonical_object_rows(ref_M, ref_M_not)
    assert np.array_equal(a, b), what + " M differs"
    assert np.array_equal(an, bn), what + " M_not differs"
