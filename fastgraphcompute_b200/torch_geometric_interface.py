"""row_splits <-> PyTorch-Geometric style ``batch`` vectors, on whatever device the input lives on
(counterparts of fastgraphcompute/torch_geometric_interface.py:4-74 of the reference).

``row_splits`` [n_events + 1] delimits events in a concatenated point list; ``batch`` [n_points]
names the event of every point.  "Strict" means the points of one event are contiguous and the
event ids do not decrease.
"""
import torch


def row_splits_from_strict_batch(batch: torch.Tensor) -> torch.Tensor:
    """int64 row splits of a contiguous batch vector, e.g. [0,0,0,1,1,2,2,2] -> [0,3,5,8].

    A new event starts wherever the id changes (ids need not be consecutive); the result stays
    on the device of ``batch``."""
    n = batch.shape[0]
    dev = batch.device
    change = torch.nonzero(batch[1:] != batch[:-1]).flatten() + 1
    return torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), change.to(torch.int64),
                      torch.full((1,), n, dtype=torch.int64, device=dev)])


def strict_batch_from_row_splits(row_splits: torch.Tensor) -> torch.Tensor:
    """int64 batch vector of row splits, e.g. [0,3,5,8] -> [0,0,0,1,1,2,2,2]."""
    rs = row_splits.to(torch.int64)
    lengths = rs[1:] - rs[:-1]
    return torch.repeat_interleave(torch.arange(lengths.shape[0], dtype=torch.int64, device=rs.device), lengths)


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
