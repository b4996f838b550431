"""Pins of the CPU oracle (oracle/fgc_oracle.c): it must reproduce
 (a) the known answers of the reference's own unit tests,
 (b) the golden vectors produced by running the reference's unmodified CPU ops
     (tests/golden/make_golden.py), and
 (c) when oracle/_ref is present, the live reference ops on fresh inputs.
CPU only.
"""
import os

import numpy as np
import pytest

from oracle import oracle
import parity


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    cases = {}
    for key in z.files:
        parts = key.split("/")
        cases.setdefault(parts[0], {}).setdefault(parts[1], {})[parts[2]] = z[key]
    return cases


# ---- (a) known answers held by the reference's tests ------------------------------------------

def test_binning_known_answer_simple():
    # tests/test_bin_by_coordinates.py:26-75 of the reference
    coords = np.array([[0.1, 0.1], [2.5, 2.5], [4.9, 4.9]], np.float32)
    b, flat, nb, bw, nper = oracle.bin_by_coordinates(coords, [0, 3], np.array([0.5], np.float32), [10, 10])
    assert b.tolist() == [[0, 0, 0], [0, 4, 4], [0, 9, 9]]
    assert flat.tolist() == [0, 44, 99]
    exp = np.zeros(100, np.int64)
    exp[[0, 44, 99]] = 1
    assert np.array_equal(nper, exp)


def test_binning_known_answer_out_of_bounds():
    # tests/test_bin_by_coordinates.py:111-155 of the reference
    coords = np.array([[-1.0, -1.0], [5.1, 5.1], [0.7, 0.7]], np.float32)
    b, flat, nb, bw, nper = oracle.bin_by_coordinates(coords, [0, 3], np.array([0.5], np.float32), [10, 10])
    assert b.tolist() == [[0, 0, 0], [0, 9, 9], [0, 3, 3]]
    assert flat.tolist() == [0, 99, 33]
    assert nper.sum() == 3 and nper[0] == 1 and nper[99] == 1 and nper[33] == 1


INDEX_REPLACER_EXPECTED = [
    [-1, 13, 57, -1, 62], [31, 54, 16, -1, 75], [66, 19, 14, 20, 36], [46, 32, 44, 79, -1],
    [23, 11, 4, 72, 93], [61, 83, 27, 65, 50], [91, 92, 71, 1, 43], [89, 53, 10, 63, 7],
    [96, 6, 24, 64, 40], [15, 94, -1, 82, 68], [86, 90, -1, -1, 41], [97, 37, 70, 80, 78],
    [21, 58, 12, 28, 9], [22, 33, 51, 73, 55], [67, 76, -1, 25, 45], [85, 30, 38, 87, 81],
    [47, 69, 49, 48, 18], [17, 2, 74, 39, -1], [59, 84, 98, 95, 88], [29, 34, 60, 52, -1]]


def index_replacer_reference_inputs():
    """Inputs of the reference's golden test (tests/test_index_replacer.py:13-32)."""
    np.random.seed(34)
    tbr = np.arange(100)
    tbr[np.random.choice(100, 10, replace=False)] = -1
    np.random.shuffle(tbr)
    tbr = tbr.reshape(20, 5)
    rpl = np.arange(100)
    np.random.shuffle(rpl)
    return tbr.astype(np.int64), rpl.astype(np.int64)


def test_index_replacer_known_answer():
    tbr, rpl = index_replacer_reference_inputs()
    out = oracle.index_replacer(tbr, rpl)
    assert out.tolist() == INDEX_REPLACER_EXPECTED


def test_knn_against_brute_force_like_reference_tests():
    # shape of tests/test_binned_select_knn.py:95-163 (seed 45, 3 row splits, K=50), smaller N
    import torch
    torch.manual_seed(45)
    n = 2000
    coords = torch.rand((n, 3)).numpy()
    rs = np.array([0, n // 3, n // 2, n])
    idx, dist = oracle.binned_select_knn(50, coords, rs)
    bidx, bdist = parity.brute_force_knn(coords, rs, 50)
    st = parity.assert_knn_parity(idx, dist, bidx, bdist, what="oracle vs brute force")
    assert st["max_rel"] == 0.0


# ---- (b) golden vectors from the reference's CPU ops -------------------------------------------

def test_knn_golden(golden_dir):
    cases = load(golden_dir, "knn")
    assert len(cases) >= 15
    for name, c in cases.items():
        i = c["in"]
        kw = {}
        if "n_bins" in i:
            kw["n_bins"] = i["n_bins"]
        if "direction" in i:
            kw["direction"] = i["direction"]
        if "max_bin_dims" in i:
            kw["max_bin_dims"] = int(i["max_bin_dims"])
        tf = bool(i["tf_compat"]) if "tf_compat" in i else False
        idx, dist = oracle.binned_select_knn(int(i["K"]), i["coords"], i["row_splits"],
                                             torch_compatible_indices=tf, **kw)
        # Same algorithm; the slot order inside a row depends on the order of equal keys in
        # the reference's (unstable) argsort, so rows are compared as sets.  Distances must
        # be bit-identical.
        ref_idx = c["out"]["idx"].astype(np.int64)
        st = parity.assert_knn_parity(idx, dist, ref_idx, c["out"]["distsq"], pad_self=tf, what=name)
        assert st["max_rel"] == 0.0, name
        if "grad" in i:
            # gradient oracle on the reference's own slot order: bit-identical
            g = oracle.binned_select_knn_grad(c["out"]["grad_dist_slots"], ref_idx, i["coords"])
            assert np.array_equal(g, c["out"]["grad_coords"]), name


def test_binning_golden(golden_dir):
    cases = load(golden_dir, "binning")
    assert "bbc_fixture" in cases
    for name, c in cases.items():
        i = c["in"]
        r = oracle.bin_by_coordinates(i["coords"], i["row_splits"], i.get("bin_width"), i.get("n_bins"),
                                      True, bool(i["pre_normalized"]) if "pre_normalized" in i else False)
        for got, key in zip(r, ("bin_indices", "flat", "n_bins", "bin_width", "n_per_bin")):
            assert np.array_equal(got, c["out"][key]), (name, key)


def test_index_replacer_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "misc.npz"))
    assert np.array_equal(oracle.index_replacer(z["ir_in"], z["ir_repl"]), z["ir_out"])


def test_gravnet_aggregate_golden(golden_dir):
    """The aggregation oracle against the reference module's recorded output: recompute
    mean/max from the recorded kNN result and push them through the recorded Linear."""
    cases = load(golden_dir, "gravnet")
    for name, c in cases.items():
        w = c["weights"]
        x = c["in"]["x"]
        prop = x @ w["propagate_transformations.weight"].T + w["propagate_transformations.bias"]
        idx = c["out"]["idx"].astype(np.int64)
        mean, mx, _ = oracle.gravnet_aggregate_fwd(prop.astype(np.float32), idx, c["out"]["distsq"])
        feat = np.concatenate([x, mean, mx], 1)
        out = feat @ w["output_transformations.0.weight"].T + w["output_transformations.0.bias"]
        out = np.maximum(out, 0)
        np.testing.assert_allclose(out, c["out"]["out"], rtol=2e-4, atol=2e-5, err_msg=name)


# ---- (c) live reference, when it was built here -------------------------------------------------

def _ref():
    from oracle import ref_ops
    if not ref_ops.available():
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    return ref_ops


def test_knn_live_reference_fresh_inputs():
    ref_ops = _ref()
    import torch
    for seed, n, d, k in ((101, 1500, 3, 20), (102, 800, 4, 33), (103, 600, 6, 9)):
        g = torch.Generator().manual_seed(seed)
        coords = torch.randn((n, d), generator=g)
        rs = torch.tensor([0, n // 4, n])
        ridx, rdist = ref_ops.ref_binned_select_knn(k, coords, rs)
        idx, dist = oracle.binned_select_knn(k, coords.numpy(), rs.numpy())
        st = parity.assert_knn_parity(idx, dist, ridx.numpy(), rdist.numpy(), what="live %d" % seed)
        assert st["max_rel"] == 0.0


def test_knn_grad_live_reference():
    ref_ops = _ref()
    import torch
    g = torch.Generator().manual_seed(7)
    coords = torch.rand((700, 3), generator=g, requires_grad=True)
    rs = torch.tensor([0, 700])
    idx, dist = ref_ops.ref_binned_select_knn(12, coords, rs)
    up = torch.randn(dist.shape, generator=g)
    (dist * up).sum().backward()
    mine = oracle.binned_select_knn_grad(up.numpy(), idx.numpy(), coords.detach().numpy())
    assert np.array_equal(mine, coords.grad.numpy())


def test_gravnet_backward_oracle_matches_autograd():
    import torch
    g = torch.Generator().manual_seed(3)
    n, k, p = 300, 12, 10
    prop = torch.randn((n, p), generator=g, requires_grad=True)
    dsq = (torch.rand((n, k), generator=g) * 0.2).requires_grad_(True)
    idx = torch.randint(0, n, (n, k), generator=g)
    idx[torch.rand((n, k), generator=g) < 0.1] = -1
    from oracle import ref_ops
    fmean, fmax = ref_ops.ref_gravnet_aggregate(prop, idx, dsq)
    gm = torch.randn(fmean.shape, generator=g)
    gx = torch.randn(fmax.shape, generator=g)
    ((fmean * gm).sum() + (fmax * gx).sum()).backward()
    mean, mx, am = oracle.gravnet_aggregate_fwd(prop.detach().numpy(), idx.numpy(), dsq.detach().numpy())
    np.testing.assert_allclose(mean, fmean.detach().numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(mx, fmax.detach().numpy(), rtol=1e-6, atol=0)
    dp, dd = oracle.gravnet_aggregate_bwd(prop.detach().numpy(), idx.numpy(), dsq.detach().numpy(), am,
                                          gm.numpy(), gx.numpy())
    parity.assert_grad_close(dp, prop.grad.numpy(), 1e-5, "d_prop")
    parity.assert_grad_close(dd, dsq.grad.numpy(), 1e-5, "d_distsq")


# ---- oc_helper_matrices --------------------------------------------------------------------

OC_KNOWN_ASSO = [3, 7, 3, -1, -1, 3, 7, 1, 1, 0, 0, -1, 1, 1, -1, 3, -1, 19, 3, 2, -1, 19]
OC_KNOWN_RS = [0, 15, 22]
OC_KNOWN_M = [[0, 2, 5, -1], [1, 6, -1, -1], [7, 8, 12, 13], [9, 10, -1, -1],
              [15, 18, -1, -1], [17, 21, -1, -1], [19, -1, -1, -1]]


def oc_known_m_not():
    """M_not of the reference's known-answer case (tests/test_oc_helper.py:88-112): every point
    of the object's row split that is not in the object, ascending, padded to 15."""
    rows = []
    for members in OC_KNOWN_M:
        first = members[0]
        lo, hi = (0, 15) if first < 15 else (15, 22)
        others = [i for i in range(lo, hi) if i not in members]
        rows.append(others + [-1] * (15 - len(others)))
    return rows


def test_oc_helper_known_answer():
    """tests/test_oc_helper.py:28-125 of the reference."""
    M, M_not, per = oracle.oc_helper_matrices(OC_KNOWN_ASSO, OC_KNOWN_RS)
    assert M.shape == (7, 4) and M_not.shape == (7, 15)
    parity.assert_oc_matrices_equal(M, M_not, per, OC_KNOWN_M, oc_known_m_not(), [4, 3], "known answer")


def test_oc_helper_golden(golden_dir):
    for name, c in load(golden_dir, "oc").items():
        M, M_not, per = oracle.oc_helper_matrices(c["in"]["asso"], c["in"]["row_splits"])
        parity.assert_oc_matrices_equal(M, M_not, per, c["out"]["M"], c["out"]["M_not"], c["out"]["per_split"], name)
        M2, M_not2, _ = oracle.oc_helper_matrices(c["in"]["asso"], c["in"]["row_splits"], calc_m_not=False)
        assert np.array_equal(M2, M) and (M_not2 == -1).all()


def test_oc_helper_live_reference():
    from oracle import ref_ops
    if not ref_ops.oc_available():
        pytest.skip("oracle/_ref/oc_helper_*.so not built (needs the reference checkout)")
    import torch
    rng = np.random.RandomState(5)
    for trial in range(10):
        sizes = [int(rng.randint(0, 80)) for _ in range(rng.randint(1, 5))]
        if sum(sizes) == 0:
            sizes[0] = 4
        rs = np.concatenate([[0], np.cumsum(sizes)])
        asso = rng.randint(-2, 9, size=int(rs[-1])).astype(np.int64)
        M, M_not, per = oracle.oc_helper_matrices(asso, rs)
        rM, rM_not, rper = ref_ops.ref_oc_helper_matrices(torch.tensor(asso), torch.tensor(rs))
        assert np.array_equal(M, rM.numpy()) and np.array_equal(M_not, rM_not.numpy())
        assert np.array_equal(per, rper.numpy())


# ---- brute-force select_knn with a radius -----------------------------------------------------

def test_select_knn_golden(golden_dir):
    for name, c in load(golden_dir, "select").items():
        i = c["in"]
        idx, dist = oracle.select_knn(int(i["K"]), i["coords"], i["row_splits"], float(i["max_radius"]))
        assert np.array_equal(idx, c["out"]["idx"].astype(np.int64)), name     # slot order included
        assert np.array_equal(dist, c["out"]["distsq"]), name


def test_select_knn_live_reference():
    from oracle import ref_ops
    if not ref_ops.select_knn_available():
        pytest.skip("oracle/_ref/select_knn_lib.so not built (needs the reference checkout)")
    import torch
    rng = np.random.RandomState(17)
    for trial in range(8):
        n = int(rng.randint(5, 200))
        c = rng.rand(n, int(rng.randint(2, 5))).astype(np.float32)
        rs = np.array([0, n // 3, n], np.int64)
        k, r = int(rng.choice([2, 7, 16])), float(rng.choice([-1.0, 0.2, 0.5]))
        idx, dist = oracle.select_knn(k, c, rs, r)
        ri, rd = ref_ops.ref_select_knn(k, torch.tensor(c), torch.tensor(rs), r)
        assert np.array_equal(idx, ri.numpy()) and np.array_equal(dist, rd.numpy())
