"""GPU parity of oc_helper_matrices and select_with_default (the consumers of the same
row_splits data on the loss side) against the reference's known answers, the golden vectors of
its CPU ops, and the CPU oracle on seeded random inputs.  Index work: bit-exact."""
import numpy as np
import pytest
import torch

import parity
from oracle import oracle
from test_oracle_pins import load, OC_KNOWN_ASSO, OC_KNOWN_RS, OC_KNOWN_M, oc_known_m_not

pytestmark = pytest.mark.gpu

import fastgraphcompute_b200 as fgc  # noqa: E402

DEV = "cuda:0"


def run(asso, rs, calc_m_not=True):
    M, M_not, per = fgc.oc_helper_matrices(torch.as_tensor(np.asarray(asso), dtype=torch.int64).to(DEV),
                                           torch.as_tensor(np.asarray(rs), dtype=torch.int64).to(DEV), calc_m_not)
    assert M.dtype == torch.int64 and M_not.dtype == torch.int64 and per.dtype == torch.int64
    assert M.is_cuda and M_not.is_cuda and per.is_cuda
    return M.cpu().numpy(), M_not.cpu().numpy(), per.cpu().numpy()


def test_known_answer_of_the_reference_test():
    """tests/test_oc_helper.py:28-125 of the reference."""
    M, M_not, per = run(OC_KNOWN_ASSO, OC_KNOWN_RS)
    assert M.shape == (7, 4) and M_not.shape == (7, 15)
    parity.assert_oc_matrices_equal(M, M_not, per, OC_KNOWN_M, oc_known_m_not(), [4, 3], "known answer")


def test_golden(golden_dir):
    for name, c in load(golden_dir, "oc").items():
        M, M_not, per = run(c["in"]["asso"], c["in"]["row_splits"])
        parity.assert_oc_matrices_equal(M, M_not, per, c["out"]["M"], c["out"]["M_not"], c["out"]["per_split"], name)
        M2, M_not2, per2 = run(c["in"]["asso"], c["in"]["row_splits"], calc_m_not=False)
        assert np.array_equal(M2, M) and (M_not2 == -1).all() and M_not2.shape == M_not.shape
        assert np.array_equal(per2, per)


def test_random_against_oracle_and_reproducible():
    rng = np.random.RandomState(11)
    for trial in range(25):
        sizes = [int(rng.choice([0, 1, rng.randint(2, 50), rng.randint(50, 3000)])) for _ in range(rng.randint(1, 6))]
        if sum(sizes) == 0:
            sizes[-1] = 7
        rs = np.concatenate([[0], np.cumsum(sizes)])
        hi = int(rng.choice([1, 3, 20, 400]))
        asso = rng.randint(-2, hi, size=int(rs[-1])).astype(np.int64)
        if trial % 4 == 0:
            asso[asso >= 0] *= 2 ** 40 + 3
        a = run(asso, rs)
        b = run(asso, rs)
        for x, y in zip(a, b):
            assert np.array_equal(x, y)          # same rows in the same order on every run
        parity.assert_oc_matrices_equal(*a, *oracle.oc_helper_matrices(asso, rs), "random %d" % trial)
        # rows come ordered by (truth index, row split)
        first = a[0][:, 0] if a[0].shape[1] else np.zeros(0, np.int64)
        keys = [(int(asso[i]), int(np.searchsorted(rs, i, side="right") - 1)) for i in first]
        assert keys == sorted(keys)


def test_edge_cases():
    M, M_not, per = run([-1, -5, -1], [0, 3])               # no object at all
    assert M.shape == (0, 0) and M_not.shape == (0, 3) and per.tolist() == [0]
    M, M_not, per = run([4, 4, 4, 4], [0, 4])                # one object owns its whole row split
    assert M.tolist() == [[0, 1, 2, 3]] and M_not.tolist() == [[-1, -1, -1, -1]] and per.tolist() == [1]
    with pytest.raises(RuntimeError):
        fgc.oc_helper_matrices(torch.zeros(5, dtype=torch.int64, device=DEV),
                               torch.tensor([0, 3], dtype=torch.int64, device=DEV))   # does not end at V
    with pytest.raises(RuntimeError):
        fgc.oc_helper_matrices(torch.zeros(5, dtype=torch.int64), torch.tensor([0, 5]))   # CPU tensors


def test_full_size_properties():
    """16 row splits of 100 000 points, 200 objects each plus noise: every row of M holds exactly the
    points of one (row split, truth index) pair, M_not holds the rest of that row split, ascending."""
    g = torch.Generator().manual_seed(3)
    n_splits, per = 16, 100000
    asso = torch.randint(-20, 200, (n_splits * per,), generator=g)
    rs = torch.arange(0, n_splits * per + 1, per)
    M, M_not, ops = fgc.oc_helper_matrices(asso.to(DEV), rs.to(DEV))
    assert ops.tolist() == [200] * n_splits and M.shape[0] == 200 * n_splits and M_not.shape[1] == per
    ad = asso.to(DEV)
    valid = M >= 0
    first = M[:, 0]
    vals = ad[first]
    # members: same truth index as the first member, same row split, ascending, counts add up
    assert bool(((ad[M.clamp(min=0)] == vals[:, None]) | ~valid).all())
    assert bool((((M // per) == (first // per)[:, None]) | ~valid).all())
    assert bool(((M[:, 1:] > M[:, :-1]) | ~valid[:, 1:]).all())
    assert int(valid.sum()) == int((asso >= 0).sum())
    nvalid = M_not >= 0
    assert bool(((ad[M_not.clamp(min=0)] != vals[:, None]) | ~nvalid).all())
    assert bool((((M_not // per) == (first // per)[:, None]) | ~nvalid).all())
    assert bool(((M_not[:, 1:] > M_not[:, :-1]) | ~nvalid[:, 1:]).all())
    assert bool((valid.sum(1) + nvalid.sum(1) == per).all())


def test_select_with_default_kernel():
    rng = np.random.RandomState(2)
    for dtype, default in ((np.float32, 0.0), (np.float32, -7.5), (np.int64, -1), (np.float64, 2.25), (np.int32, 9)):
        for v, k, f, n in ((50, 7, 3, 50), (200, 16, 1, 120), (33, 4, 32, 64), (0, 5, 3, 10)):
            idx = rng.randint(-1, n, size=(v, k)).astype(np.int64)
            feat = (rng.randn(n, f) * 100).astype(dtype)
            out = fgc.select_with_default(torch.as_tensor(idx).to(DEV), torch.as_tensor(feat).to(DEV), default)
            assert out.shape == (v, k, f) and out.dtype == torch.as_tensor(feat).dtype
            assert np.array_equal(out.cpu().numpy(), oracle.select_with_default(idx, feat, default))
    # the reference's own use: point ids through M (object_condensation.py:148)
    M, _, _ = fgc.oc_helper_matrices(torch.tensor(OC_KNOWN_ASSO, device=DEV), torch.tensor(OC_KNOWN_RS, device=DEV))
    ids = torch.arange(len(OC_KNOWN_ASSO), device=DEV, dtype=torch.int64).view(-1, 1)
    assert torch.equal(fgc.select_with_default(M, ids, -1)[:, :, 0], M)


def test_select_with_default_gradient():
    g = torch.Generator().manual_seed(8)
    idx = torch.randint(-1, 40, (60, 9), generator=g).to(DEV)
    feat = torch.randn((40, 5), generator=g).to(DEV).requires_grad_(True)
    up = torch.randn((60, 9, 5), generator=g).to(DEV)
    (fgc.select_with_default(idx, feat, 0.0) * up).sum().backward()
    ref = torch.zeros((40, 5), dtype=torch.float64)
    ic, uc = idx.cpu(), up.cpu().double()
    for a in range(60):
        for b in range(9):
            if ic[a, b] >= 0:
                ref[ic[a, b]] += uc[a, b]
    parity.assert_grad_close(feat.grad.cpu().numpy(), ref.numpy(), what="select_with_default grad")
