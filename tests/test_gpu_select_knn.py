"""GPU parity of select_knn (k nearest neighbours within a radius; the reference's brute-force op
select_knn::select_knn) against the golden vectors of its CPU kernel and the CPU oracle.
Rows are compared as sets (parity.assert_knn_parity): index sets exact up to 1-ulp ties at the
K-th distance, squared distances within 1e-6 relative (measured: bit-identical)."""
import numpy as np
import pytest
import torch

import parity
from oracle import oracle
from test_oracle_pins import load

pytestmark = pytest.mark.gpu

import fastgraphcompute_b200 as fgc  # noqa: E402

DEV = "cuda:0"


def test_golden(golden_dir):
    for name, c in load(golden_dir, "select").items():
        i = c["in"]
        idx, dist = fgc.select_knn(int(i["K"]), torch.as_tensor(i["coords"]).to(DEV),
                                   torch.as_tensor(i["row_splits"]).to(DEV), max_radius=float(i["max_radius"]))
        assert idx.dtype == torch.int64 and dist.dtype == torch.float32
        st = parity.assert_knn_parity(idx.cpu().numpy(), dist.cpu().numpy(), c["out"]["idx"], c["out"]["distsq"],
                                      what=name)
        assert st["max_rel"] == 0.0


def test_random_against_oracle_with_gradient():
    rng = np.random.RandomState(23)
    for trial in range(30):
        sizes = [int(rng.choice([0, 1, rng.randint(2, 30), rng.randint(30, 700)])) for _ in range(rng.randint(1, 5))]
        if sum(sizes) == 0:
            sizes[0] = 6
        rs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        d = int(rng.randint(2, 6))
        k = int(rng.choice([1, 4, 16, 33, 70]))
        c = rng.rand(int(rs[-1]), d).astype(np.float32)
        r = float(rng.choice([-1.0, 0.05, 0.2, 0.6, 3.0]))
        what = "select case %d (N=%d D=%d K=%d r=%g)" % (trial, c.shape[0], d, k, r)
        coords = torch.as_tensor(c).to(DEV).requires_grad_(True)
        idx, dist = fgc.select_knn(k, coords, torch.as_tensor(rs).to(DEV), max_radius=r)
        oi, od = oracle.select_knn(k, c, rs, r)
        parity.assert_knn_parity(idx.cpu().numpy(), dist.detach().cpu().numpy(), oi, od, what=what)
        if r > 0:
            r2 = np.float32(r * r)
            assert bool((dist.detach().cpu().numpy() <= r2).all())
        up = rng.randn(c.shape[0], k).astype(np.float32)
        (dist * torch.as_tensor(up).to(DEV)).sum().backward()
        og = oracle.binned_select_knn_grad(up, idx.cpu().numpy(), c)
        parity.assert_grad_close(coords.grad.cpu().numpy(), og, what=what + " grad")


def test_radius_filter_entry_point_in_place():
    """fgc_knn_radius_filter on hand-made rows: kept slots close up in order, pads follow."""
    from fastgraphcompute_b200 import _cabi
    idx = torch.tensor([[0, 5, 7, -1, -1], [1, 9, 3, 4, 2], [2, 2, 2, 2, 2]], dtype=torch.int64, device=DEV)
    dist = torch.tensor([[0., 0.5, 0.04, 0., 0.], [0., 0.01, 0.3, 0.02, 0.09], [0., 0., 0., 0., 0.]], device=DEV)
    st = _cabi.current_stream(idx.device)
    a, b = idx[:2].clone(), dist[:2].clone()
    assert _cabi.lib.fgc_knn_radius_filter(_cabi.ptr(a), _cabi.ptr(b), 2, 5, 0.3, 0, st) == 0
    assert a.tolist() == [[0, 7, -1, -1, -1], [1, 9, 4, 2, -1]]
    assert torch.allclose(b, torch.tensor([[0., 0.04, 0., 0., 0.], [0., 0.01, 0.02, 0.09, 0.]], device=DEV))
    a, b = idx.clone(), dist.clone()          # pads written as the point itself
    assert _cabi.lib.fgc_knn_radius_filter(_cabi.ptr(a), _cabi.ptr(b), 3, 5, 0.3, 1, st) == 0
    assert a.tolist() == [[0, 7, 0, 0, 0], [1, 9, 4, 2, 1], [2, 2, 2, 2, 2]]
    a, b = idx.clone(), dist.clone()          # no radius: untouched
    assert _cabi.lib.fgc_knn_radius_filter(_cabi.ptr(a), _cabi.ptr(b), 3, 5, -1.0, 0, st) == 0
    assert torch.equal(a, idx) and torch.equal(b, dist)
