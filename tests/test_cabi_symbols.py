"""The C-ABI library loads and exports every function include/fgc_b200.h declares (CPU only:
no compute call is made)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fgc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fgc_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path():
    names = declared_functions()
    for must in ("fgc_bin_prepare", "fgc_bin_assign", "fgc_binned_knn_fwd", "fgc_binned_knn_bwd",
                 "fgc_index_replacer", "fgc_gravnet_aggregate_fwd", "fgc_gravnet_aggregate_bwd",
                 "fgc_knn_workspace_bytes", "fgc_read_status"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from fastgraphcompute_b200 import _cabi
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), "libfgc_b200.so does not export " + name
        assert name in _cabi.SIGNATURES, "python binding lacks " + name
    assert _cabi.lib.fgc_version() >= 100
    assert b"workspace" in _cabi.lib.fgc_error_string(-4)


def test_workspace_size_is_monotone_and_rejects_bad_arguments():
    from fastgraphcompute_b200 import _cabi
    f = _cabi.lib.fgc_knn_workspace_bytes
    assert f(-1, 3, 2, 8) == 0 and f(10, 0, 2, 8) == 0 and f(10, 3, 0, 8) == 0 and f(10, 3, 2, 0) == 0
    a, b = f(1000, 3, 2, 16), f(100000, 3, 2, 16)
    assert 0 < a < b
    assert f(100000, 8, 2, 16) > b


def test_bin_params_mirror_matches_header():
    from fastgraphcompute_b200 import _cabi
    assert ctypes.sizeof(_cabi.BinParams) == 256
    assert _cabi.BinParams.n_bins.offset == 48


def test_cpu_tensors_are_rejected_loudly():
    import pytest
    import torch
    import fastgraphcompute_b200 as fgc
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        fgc.binned_select_knn(4, torch.rand(10, 3), torch.tensor([0, 10]))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        fgc.bin_by_coordinates(torch.rand(10, 3), torch.tensor([0, 10]), n_bins=torch.tensor(3))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        fgc.index_replacer(torch.zeros(3, dtype=torch.int64), torch.zeros(3, dtype=torch.int64))


def test_select_with_default_matches_oracle():
    import numpy as np
    import torch
    from fastgraphcompute_b200 import select_with_default
    from oracle import oracle
    g = torch.Generator().manual_seed(0)
    idx = torch.randint(-1, 20, (20, 5), generator=g)
    for feat in (torch.randn((20, 3), generator=g), torch.randint(0, 9, (20, 2), generator=g)):
        out = select_with_default(idx, feat, -7.0)
        assert out.dtype == feat.dtype and out.shape == (20, 5, feat.shape[1])
        assert np.array_equal(out.numpy(), oracle.select_with_default(idx.numpy(), feat.numpy(), -7.0))


def test_row_splits_batch_round_trip():
    import torch
    from fastgraphcompute_b200.torch_geometric_interface import (row_splits_from_strict_batch,
                                                                  strict_batch_from_row_splits)
    batch = torch.tensor([0, 0, 0, 1, 1, 2, 2, 2])
    rs = row_splits_from_strict_batch(batch)
    assert rs.tolist() == [0, 3, 5, 8] and rs.dtype == torch.int64
    assert torch.equal(strict_batch_from_row_splits(rs), batch)
    assert strict_batch_from_row_splits(torch.tensor([0, 2, 2, 5], dtype=torch.int32)).tolist() == [0, 0, 2, 2, 2]
    assert row_splits_from_strict_batch(torch.tensor([4, 4, 7])).tolist() == [0, 2, 3]
