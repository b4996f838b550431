"""Input definitions of the golden parity cases (shared by make_golden.py and the tests).

Every case is a dict of numpy arrays / scalars.  Inputs are generated from fixed
seeds here and ALSO stored in the golden files, so the committed vectors do not
depend on a random-number generator staying stable.
"""
import numpy as np
import torch


def _rand(seed, *shape):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(shape, generator=g, dtype=torch.float32).numpy()


def _randn(seed, *shape):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).numpy()


def knn_cases():
    """name -> dict(coords, row_splits, K, [n_bins], [direction], [tf_compat], [max_bin_dims], [grad])"""
    cases = {}
    n = 1500
    cases["uniform3d_k50"] = dict(coords=_rand(45, n, 3), row_splits=np.array([0, n // 3, n // 2, n]), K=50)
    n = 1000
    cases["uniform8d_k50"] = dict(coords=_rand(46, n, 8), row_splits=np.array([0, n // 3, n // 2, n]), K=50)
    for name, d, k in (("grad_d2_k5", 2, 5), ("grad_d4_k10", 4, 10), ("grad_d2_k50", 2, 50)):
        cases[name] = dict(coords=_rand(45 + d + k, 1000, d) - 0.5, row_splits=np.array([0, 1000]), K=k,
                           n_bins=np.array(10), grad=_randn(7 + k, 1000, k))
    from fastgraphcompute_b200 import synthetic
    w = synthetic.c1_two_events()
    cases["c1_two_events"] = dict(coords=w.coords.numpy(), row_splits=w.row_splits.numpy().astype(np.int64),
                                  K=w.K, n_bins=w.n_bins.numpy(), grad=w.grad_distsq.numpy())
    w = synthetic.c2_gaussian_mixture(scale=0.01)
    cases["c2_gmm_small"] = dict(coords=w.coords.numpy(), row_splits=w.row_splits.numpy(), K=w.K,
                                 grad=w.grad_distsq.numpy())
    w = synthetic.c5_skewed(scale=0.0012, n_events=2, n_clusters=12)
    cases["c5_skewed_small"] = dict(coords=w.coords.numpy(), row_splits=w.row_splits.numpy(), K=w.K)
    # events smaller than K, an empty event, and a normal one
    rs = np.array([0, 0, 6, 9, 40, 40, 700])
    cases["small_events_k8"] = dict(coords=_rand(3, 700, 3), row_splits=rs, K=8, grad=_randn(4, 700, 8))
    cases["small_events_k8_tf"] = dict(coords=_rand(3, 700, 3), row_splits=rs, K=8, tf_compat=True)
    # exact duplicates (distance 0 neighbours) and coarse lattice points (many exact ties)
    c = _rand(5, 600, 3)
    c[300:] = c[:300]
    cases["duplicates_k6"] = dict(coords=c, row_splits=np.array([0, 600]), K=6)
    g = torch.Generator().manual_seed(9)
    lattice = torch.randint(0, 12, (1500, 3), generator=g).float().numpy() * 0.125
    cases["lattice_ties_k12"] = dict(coords=lattice, row_splits=np.array([0, 700, 1500]), K=12)
    g = torch.Generator().manual_seed(11)
    direction = torch.randint(0, 4, (1500,), generator=g).numpy().astype(np.int64)
    cases["direction_k10"] = dict(coords=_rand(12, 1500, 3), row_splits=np.array([0, 600, 1500]), K=10,
                                  direction=direction, grad=_randn(13, 1500, 10))
    cases["d5_mbd5_k20"] = dict(coords=_rand(14, 1200, 5), row_splits=np.array([0, 1200]), K=20, max_bin_dims=5)
    cases["d2_k33"] = dict(coords=_rand(15, 900, 2), row_splits=np.array([0, 400, 900]), K=33)
    cases["d3_k130"] = dict(coords=_randn(16, 500, 3), row_splits=np.array([0, 500]), K=130)
    # a degenerate dimension (all equal) and detector-like magnitudes
    c = _randn(17, 800, 4) * 300.0
    c[:, 1] = 42.0
    cases["flat_dim_k16"] = dict(coords=c, row_splits=np.array([0, 800]), K=16)
    return cases


def binning_cases():
    """name -> dict(coords, row_splits, [bin_width], [n_bins], [pre_normalized])"""
    cases = {}
    rs3 = np.array([0, 300, 550, 1000])
    cases["rand2d_nbins"] = dict(coords=_randn(21, 1000, 2) * 3.0, row_splits=rs3, n_bins=np.array([7, 9]))
    cases["rand4d_scalar_nbins"] = dict(coords=_rand(22, 1000, 4) * 10.0 - 2.0, row_splits=rs3, n_bins=np.array(5))
    cases["rand3d_binwidth"] = dict(coords=_rand(23, 1000, 3) * 4.0, row_splits=rs3, bin_width=np.array([0.37], np.float32))
    cases["rand3d_prenorm"] = dict(coords=_rand(24, 1000, 3) * 2.0, row_splits=rs3, n_bins=np.array([4, 5, 6]),
                                   pre_normalized=True)
    cases["both_given_clamps"] = dict(coords=_rand(25, 500, 2) * 8.0, row_splits=np.array([0, 500]),
                                      bin_width=np.array([0.5], np.float32), n_bins=np.array([10, 10]))
    return cases


def gravnet_cases():
    """name -> dict(in_channels, propagate, space, k, out_channels, n, row_splits)"""
    rs = np.array([0, 50, 80, 100])
    return {
        "gn_in8_p8_k8_s3": dict(in_channels=8, propagate=8, space=3, k=8, out_channels=16, n=100, row_splits=rs),
        "gn_in12_p12_k32_s2": dict(in_channels=12, propagate=12, space=2, k=32, out_channels=24, n=100, row_splits=rs),
        "gn_in64_p64_k8_s5": dict(in_channels=64, propagate=64, space=5, k=8, out_channels=128, n=100, row_splits=rs),
        "gn_in16_p40_k40_s4": dict(in_channels=16, propagate=40, space=4, k=40, out_channels=8, n=600,
                                   row_splits=np.array([0, 250, 600])),
    }
