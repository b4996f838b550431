"""Seeded synthetic workloads of the hot path (CPU tensors; copy to the GPU to use).

One generator per benchmark configuration, shared by the parity tests, the smoke
check and the benchmark so that every leg sees identical inputs.  ``scale``
shrinks the point counts (event sizes are multiplied by it) for test-sized runs;
scale=1 is the full configuration.
"""
import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class KnnWorkload:
    name: str
    coords: torch.Tensor              # [N, D] float32
    row_splits: torch.Tensor          # [n_events + 1]
    K: int
    n_bins: Optional[torch.Tensor] = None   # what the reference is asked to use (None: its default)
    grad_distsq: Optional[torch.Tensor] = None  # upstream gradient on distsq, [N, K]

    @property
    def n_points(self):
        return int(self.coords.shape[0])


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def c1_two_events(scale=1.0, seed=0):
    """10 000 uniform points in [0,1)^3, two events of 5 000, K=16, 7 bins per dimension."""
    g = _gen(seed)
    per = max(int(5000 * scale), 20)
    n = 2 * per
    coords = torch.rand((n, 3), generator=g, dtype=torch.float32)
    rs = torch.tensor([0, per, n], dtype=torch.int32)
    K = 16
    nb = int(math.ceil((per / K) ** (1.0 / 3.0)))
    grad = torch.randn((n, K), generator=g, dtype=torch.float32)
    return KnnWorkload("c1_two_events", coords, rs, K, torch.tensor(nb, dtype=torch.int64), grad)


def c2_gaussian_mixture(scale=1.0, seed=0):
    """Single event, 200 000 points in 4-D from 50 Gaussians (sigma 0.02, centres uniform), K=32."""
    g = _gen(seed)
    n = max(int(200000 * scale), 64)
    centres = torch.rand((50, 4), generator=g, dtype=torch.float32)
    comp = torch.randint(0, 50, (n,), generator=g)
    coords = centres[comp] + 0.02 * torch.randn((n, 4), generator=g, dtype=torch.float32)
    rs = torch.tensor([0, n], dtype=torch.int64)
    K = 32
    grad = torch.randn((n, K), generator=g, dtype=torch.float32)
    return KnnWorkload("c2_gaussian_mixture", coords.contiguous(), rs, K, None, grad)


def c3_event_batch(scale=1.0, seed=0, n_events=64):
    """64 events of 50 000..150 000 uniform points in [0,1)^3, K=64, int32 row splits."""
    g = _gen(seed)
    sizes = torch.randint(50000, 150001, (n_events,), generator=g)
    sizes = torch.clamp((sizes.double() * scale).long(), min=8)
    n = int(sizes.sum())
    coords = torch.rand((n, 3), generator=g, dtype=torch.float32)
    rs = torch.zeros(n_events + 1, dtype=torch.int32)
    rs[1:] = torch.cumsum(sizes, 0).to(torch.int32)
    return KnnWorkload("c3_event_batch", coords, rs, 64, None, None)


def c5_skewed(scale=1.0, seed=0, n_events=8, n_clusters=200):
    """8 events of 1 000 000 points in 3-D: 90 % in Gaussian clusters (sigma 0.005, Pareto(1.5)
    cluster sizes, centres uniform), 10 % uniform background; K=128."""
    g = _gen(seed)
    per = max(int(1000000 * scale), 256)
    parts = []
    for _ in range(n_events):
        centres = torch.rand((n_clusters, 3), generator=g, dtype=torch.float32)
        u = torch.rand((n_clusters,), generator=g, dtype=torch.float64)
        weights = (1.0 - u).pow(-1.0 / 1.5)            # Pareto(alpha = 1.5), x_m = 1
        n_cl = int(0.9 * per)
        sizes = torch.floor(weights / weights.sum() * n_cl).long()
        sizes[0] += n_cl - int(sizes.sum())
        comp = torch.repeat_interleave(torch.arange(n_clusters), sizes)
        pts = centres[comp] + 0.005 * torch.randn((n_cl, 3), generator=g, dtype=torch.float32)
        bg = torch.rand((per - n_cl, 3), generator=g, dtype=torch.float32)
        ev = torch.cat([pts, bg], 0)
        ev = ev[torch.randperm(per, generator=g)]
        parts.append(ev)
    coords = torch.cat(parts, 0).contiguous()
    rs = torch.arange(0, n_events + 1, dtype=torch.int64) * per
    return KnnWorkload("c5_skewed", coords, rs, 128, None, None)


@dataclass
class GravNetWorkload:
    name: str
    x: torch.Tensor            # [N, in_channels]
    row_splits: torch.Tensor
    in_channels: int
    out_channels: int
    space_dimensions: int
    propagate_dimensions: int
    k: int
    seed: int


def c4_gravnet(scale=1.0, seed=0, n_events=16):
    """GravNetOp(64 -> 64, space 4, propagate 32, k 40) on 16 events of 100 000 points, x ~ N(0,1)."""
    g = _gen(seed)
    per = max(int(100000 * scale), 50)
    n = n_events * per
    x = torch.randn((n, 64), generator=g, dtype=torch.float32)
    rs = torch.arange(0, n_events + 1, dtype=torch.int64) * per
    return GravNetWorkload("c4_gravnet", x, rs, 64, 64, 4, 32, 40, seed)


def init_gravnet_weights(module, seed=0):
    """Xavier-uniform weights for the three Linear layers (biases keep their defaults),
    seeded so that any GravNetOp-shaped module gets identical parameters."""
    g = _gen(seed + 1000)
    with torch.no_grad():
        for lin in (module.space_transformations, module.propagate_transformations,
                    module.output_transformations[0]):
            fan_out, fan_in = lin.weight.shape
            bound = math.sqrt(6.0 / (fan_in + fan_out))
            w = (torch.rand(lin.weight.shape, generator=g, dtype=torch.float32) * 2 - 1) * bound
            lin.weight.copy_(w.to(lin.weight.device))
            b = (torch.rand(lin.bias.shape, generator=g, dtype=torch.float32) * 2 - 1) / math.sqrt(fan_in)
            lin.bias.copy_(b.to(lin.bias.device))
    return module
