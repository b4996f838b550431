"""The allocation-free kNN entry point (fgc_binned_knn_fwd_static) against the regular one.

Some hosts of this library may not allocate device memory when they call it (fixed memory
budgets, plugins that only get input/output pointers); for them the library carries a fixed
scratch area.  This test drives that entry point through the C ABI twice in a row -- the
second call finds the first call's leftovers in the shared area -- and compares each result
with fgc_binned_knn_fwd on the same inputs under the kNN parity rule (identical neighbour
sets up to 1-ulp ties, squared distances within 1e-6 relative).  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

import parity
from oracle import oracle

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _regular(cabi, coords, rs, K, direction, tf):
    n, d = coords.shape
    idx = torch.empty((n, K), dtype=torch.int64, device=DEV)
    dsq = torch.empty((n, K), dtype=torch.float32, device=DEV)
    nbytes = cabi.lib.fgc_knn_workspace_bytes(n, d, rs.numel(), K)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    rc = cabi.lib.fgc_binned_knn_fwd(cabi.ptr(coords), n, d, cabi.ptr(rs), rs.numel(), K, cabi.ptr(direction),
                                     int(tf), 0.0, cabi.ptr(idx), cabi.ptr(dsq), cabi.ptr(ws), nbytes,
                                     cabi.current_stream(coords.device))
    assert rc == 0
    return idx, dsq, int(ws[:4].view(torch.int32).item())


def _static(cabi, coords, rs, K, direction, tf):
    n, d = coords.shape
    idx = torch.full((n, K), -7, dtype=torch.int64, device=DEV)
    dsq = torch.full((n, K), -7.0, dtype=torch.float32, device=DEV)
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rc = cabi.lib.fgc_binned_knn_fwd_static(cabi.ptr(coords), n, d, cabi.ptr(rs), rs.numel(), K,
                                            cabi.ptr(direction), int(tf), 0.0, cabi.ptr(idx), cabi.ptr(dsq),
                                            cabi.ptr(status), cabi.current_stream(coords.device))
    return rc, idx, dsq, status


def test_static_scratch_entry_point_matches_regular_one_twice():
    from fastgraphcompute_b200 import _cabi as cabi
    g = torch.Generator().manual_seed(123)
    cases = [
        # (n, d, row splits, K, with direction, tf_compat)
        (20000, 3, [0, 7000, 7000, 20000], 24, False, False),
        (9000, 5, [0, 40, 9000], 40, True, True),       # different shape: stale grid of call 1 is larger
    ]
    with torch.cuda.device(DEV):
        for n, d, rs_list, K, use_dir, tf in cases:
            coords = torch.randn((n, d), generator=g).to(DEV)
            rs = torch.tensor(rs_list, dtype=torch.int64, device=DEV)
            direction = torch.randint(0, 4, (n,), generator=g).to(DEV) if use_dir else None
            rc, idx, dsq, status = _static(cabi, coords, rs, K, direction, tf)
            assert rc == 0, cabi.error_string(rc)
            ridx, rdsq, rstatus = _regular(cabi, coords, rs, K, direction, tf)
            torch.cuda.synchronize()
            assert int(status.item()) == 0 and rstatus == 0
            parity.assert_knn_parity(idx.cpu().numpy(), dsq.cpu().numpy(), ridx.cpu().numpy(),
                                     rdsq.cpu().numpy(), pad_self=tf, what="static vs regular")
            # and against the CPU oracle (the regular entry point is CUDA code as well)
            oidx, odsq = oracle.binned_select_knn(
                K, coords.cpu().numpy(), rs.cpu().numpy(),
                direction=None if direction is None else direction.cpu().numpy(),
                torch_compatible_indices=tf)
            parity.assert_knn_parity(idx.cpu().numpy(), dsq.cpu().numpy(), oidx, odsq, pad_self=tf,
                                     what="static vs oracle")


def test_static_scratch_entry_point_limits_and_status():
    from fastgraphcompute_b200 import _cabi as cabi
    with torch.cuda.device(DEV):
        # beyond the built-in scratch: refused with its own error code, outputs untouched
        n = 200000
        assert cabi.lib.fgc_knn_workspace_bytes(n, 3, 2, 8) > cabi.STATIC_WORKSPACE_BYTES
        coords = torch.rand((n, 3), device=DEV)
        rs = torch.tensor([0, n], dtype=torch.int64, device=DEV)
        rc, idx, dsq, status = _static(cabi, coords, rs, 8, None, False)
        assert rc == cabi.ERR_STATIC_TOO_LARGE
        assert "scratch" in cabi.error_string(rc)
        torch.cuda.synchronize()
        assert int(idx[0, 0].item()) == -7 and int(status.item()) == -1
        # data problems still arrive through the status word
        bad = torch.rand((1000, 3), device=DEV)
        bad[5, 1] = float("nan")
        rs = torch.tensor([0, 1000], dtype=torch.int64, device=DEV)
        rc, idx, dsq, status = _static(cabi, bad, rs, 8, None, False)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) & cabi.STATUS_NONFINITE
        # nothing was searched: every row holds the defaults of a point without neighbours
        assert torch.equal(idx[:, 0], torch.arange(1000, device=DEV)) and bool((idx[:, 1:] == -1).all())
        assert float(dsq.abs().max()) == 0.0
        # and a clean call afterwards works again
        good = torch.rand((1000, 3), device=DEV)
        rc, idx, dsq, status = _static(cabi, good, rs, 8, None, False)
        ridx, rdsq, _ = _regular(cabi, good, rs, 8, None, False)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        parity.assert_knn_parity(idx.cpu().numpy(), dsq.cpu().numpy(), ridx.cpu().numpy(), rdsq.cpu().numpy())
