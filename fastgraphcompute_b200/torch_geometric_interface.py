"""row_splits <-> PyTorch-Geometric style ``batch`` vectors, on whatever device the input lives on
(counterparts of fastgraphcompute/torch_geometric_interface.py:4-74 of the reference).

``row_splits`` [n_events + 1] delimits events in a concatenated point list; ``batch`` [n_points]
names the event of every point.  "Strict" means the points of one event are contiguous and the
event ids do not decrease.
"""
import ctypes

import torch

from . import _cabi


def row_splits_from_strict_batch(batch: torch.Tensor) -> torch.Tensor:
    """int64 row splits of a contiguous batch vector, e.g. [0,0,0,1,1,2,2,2] -> [0,3,5,8].

    A new event starts wherever the id changes (ids need not be consecutive); an empty batch
    gives [0, 0].  CUDA tensors go through libfgc_b200.so (flags, scan, scatter; one host read
    for the number of events) and the result stays on their device; tensors in host memory are
    converted with the reference's own two tensor operations (this is bookkeeping beside the
    data path, where the reference's tests call it)."""
    n = batch.shape[0]
    if not batch.is_cuda:
        change = torch.nonzero(batch[1:] != batch[:-1]).flatten() + 1
        return torch.cat([torch.zeros(1, dtype=torch.int64), change.to(torch.int64),
                          torch.full((1,), n, dtype=torch.int64)])
    dev = batch.device
    b = batch.to(torch.int64).contiguous()
    out = torch.empty(n + 1 if n > 0 else 2, dtype=torch.int64, device=dev)
    nbytes = _cabi.lib.fgc_pyg_workspace_bytes(n)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    count = ctypes.c_int64(0)
    with torch.cuda.device(dev):
        stream = _cabi.current_stream(dev)
        _cabi.check(_cabi.lib.fgc_row_splits_from_strict_batch(_cabi.ptr(b), n, _cabi.ptr(out), _cabi.ptr(ws),
                                                               nbytes, stream), "fgc_row_splits_from_strict_batch")
        _cabi.check(_cabi.lib.fgc_pyg_read_count(_cabi.ptr(ws), ctypes.byref(count), stream), "fgc_pyg_read_count")
    return out[: count.value]


def strict_batch_from_row_splits(row_splits: torch.Tensor) -> torch.Tensor:
    """int64 batch vector of row splits, e.g. [0,3,5,8] -> [0,0,0,1,1,2,2,2] (one binary search
    per point on CUDA tensors; host tensors as in the reference)."""
    rs = row_splits.to(torch.int64)
    if not rs.is_cuda:
        lengths = rs[1:] - rs[:-1]
        return torch.repeat_interleave(torch.arange(lengths.shape[0], dtype=torch.int64), lengths)
    rs = rs.contiguous()
    n = int(rs[-1].item()) if rs.numel() > 0 else 0
    out = torch.empty(n, dtype=torch.int64, device=rs.device)
    if n > 0:
        with torch.cuda.device(rs.device):
            _cabi.check(_cabi.lib.fgc_strict_batch_from_row_splits(
                _cabi.ptr(rs), rs.numel(), n, _cabi.ptr(out), _cabi.current_stream(rs.device)),
                "fgc_strict_batch_from_row_splits")
    return out


class GravNetConv(torch.nn.Module):
    """GravNet layer with the call signature PyTorch-Geometric users know,
    ``layer(x, batch=None) -> out`` (how performance/gravnet_perfm.py:80-83 of the reference calls
    its torch-geometric arm), on top of GravNetOp: the strict ``batch`` vector is turned into row
    splits on the device and only the transformed features are returned.

    The parameters live in ``self.op`` (a GravNetOp, same sub-module names as the reference's)."""

    def __init__(self, in_channels: int, out_channels: int, space_dimensions: int,
                 propagate_dimensions: int, k: int):
        super().__init__()
        from .gnn_ops import GravNetOp
        self.op = GravNetOp(in_channels, out_channels, space_dimensions, propagate_dimensions, k)

    def forward(self, x: torch.Tensor, batch=None) -> torch.Tensor:
        if batch is None:
            row_splits = torch.tensor([0, x.shape[0]], dtype=torch.int64, device=x.device)
        else:
            row_splits = row_splits_from_strict_batch(batch)
        return self.op(x, row_splits)[0]
