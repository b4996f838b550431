"""row_splits <-> batch conversions against vectors recorded from the reference's own functions
(tests/golden/pyg.npz, made by tests/golden/make_golden.py pyg; the first four cases of each
direction are the inputs of the reference's tests/test_torch_geometric_interface.py:8-66).
Host tensors here, the device kernels in the GPU test below."""
import os

import numpy as np
import pytest
import torch

from fastgraphcompute_b200.torch_geometric_interface import (row_splits_from_strict_batch,
                                                             strict_batch_from_row_splits)


def _cases(golden_dir, direction):
    z = np.load(os.path.join(golden_dir, "pyg.npz"))
    names = sorted({k.split("/")[1] for k in z.files if k.startswith(direction + "/")})
    assert len(names) >= 6
    return [(n, z["%s/%s/in" % (direction, n)], z["%s/%s/out" % (direction, n)]) for n in names]


def _check(golden_dir, device):
    for name, inp, out in _cases(golden_dir, "batch_to_rs"):
        got = row_splits_from_strict_batch(torch.tensor(inp, dtype=torch.int64, device=device))
        assert got.dtype == torch.int64 and got.device.type == torch.device(device).type
        assert np.array_equal(got.cpu().numpy(), out), name
    for name, inp, out in _cases(golden_dir, "rs_to_batch"):
        got = strict_batch_from_row_splits(torch.tensor(inp, dtype=torch.int64, device=device))
        assert got.dtype == torch.int64 and got.device.type == torch.device(device).type
        assert np.array_equal(got.cpu().numpy(), out), name


def test_conversions_on_host_tensors(golden_dir):
    _check(golden_dir, "cpu")


@pytest.mark.gpu
def test_conversions_on_the_device(golden_dir):
    _check(golden_dir, "cuda:0")
    # int32 row splits (the reference's GravNet tests pass those) and a large round trip
    rs = torch.tensor([0, 5, 5, 12], dtype=torch.int32, device="cuda:0")
    assert strict_batch_from_row_splits(rs).tolist() == [0] * 5 + [2] * 7
    g = torch.Generator().manual_seed(1)
    sizes = torch.randint(0, 3000, (2000,), generator=g)
    big = torch.zeros(2001, dtype=torch.int64)
    big[1:] = torch.cumsum(sizes, 0)
    batch = strict_batch_from_row_splits(big.to("cuda:0"))
    assert torch.equal(batch.cpu(), torch.repeat_interleave(torch.arange(2000), sizes))
    back = row_splits_from_strict_batch(batch)
    keep = torch.cat([torch.tensor([True]), sizes > 0])      # empty events leave no trace in a batch vector
    assert torch.equal(back.cpu(), big[keep])
