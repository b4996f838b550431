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
