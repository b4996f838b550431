"""Stacked-GravNet model: the end-to-end workload the reference times in
performance/gravnet_perfm.py:20-96 (two dense layers, ``num_gravnet_layers`` blocks of one
GravNet layer followed by three dense layers, two dense layers at the end).

Same sub-module names and shapes as the reference's benchmark model, so a state_dict moves
between the two.  ``the_op`` is the GravNet layer class; the default is this package's
GravNetOp, called as ``layer(x, row_splits)`` like the reference's "custom" arm.
"""
from typing import Optional

import torch
from torch import nn

from .gnn_ops import GravNetOp


class GravNetModel(nn.Module):
    """forward(x [N, in_dim], row_splits [n_events + 1]) -> [N, output_dim]."""

    def __init__(self, in_dim: int, prop_dim: int, space_dim: int, k: int, hidden_dim: int,
                 output_dim: int, num_gravnet_layers: int = 4, the_op=None):
        super().__init__()
        if the_op is None:
            the_op = GravNetOp
        self.fc1 = nn.Linear(in_dim, hidden_dim)
        self.fc2 = nn.Linear(hidden_dim, hidden_dim)
        self.num_gravnet_layers = num_gravnet_layers
        self.gravnet_layers = nn.ModuleList()
        self.dense_after_gravnet = nn.ModuleList()
        for i in range(num_gravnet_layers):
            self.gravnet_layers.append(the_op(
                in_channels=hidden_dim if i == 0 else 2 * prop_dim,
                out_channels=2 * prop_dim,
                space_dimensions=space_dim,
                propagate_dimensions=prop_dim,
                k=k))
            self.dense_after_gravnet.append(nn.Sequential(
                nn.Linear(2 * prop_dim, hidden_dim), nn.ReLU(),
                nn.Linear(hidden_dim, hidden_dim), nn.ReLU(),
                nn.Linear(hidden_dim, 2 * prop_dim), nn.ReLU()))
        self.fc3 = nn.Linear(2 * prop_dim, hidden_dim)
        self.fc4 = nn.Linear(hidden_dim, output_dim)
        self.relu = nn.ReLU()

    def forward(self, x: torch.Tensor, row_splits: Optional[torch.Tensor] = None) -> torch.Tensor:
        if row_splits is None:
            row_splits = torch.tensor([0, x.shape[0]], dtype=torch.int64, device=x.device)
        x = self.relu(self.fc1(x))
        x = self.relu(self.fc2(x))
        for layer, dense in zip(self.gravnet_layers, self.dense_after_gravnet):
            x = layer(x, row_splits)[0]
            x = dense(x)
        x = self.relu(self.fc3(x))
        return self.fc4(x)
