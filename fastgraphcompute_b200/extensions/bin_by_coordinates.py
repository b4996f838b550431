"""bin_by_coordinates -- drop-in for fastgraphcompute.extensions.bin_by_coordinates.

Same signature, defaults, returned tuple, dtypes and error behaviour as the
reference wrapper (extensions/bin_by_coordinates.py:11-111); the work is done by
fgc_bin_prepare / fgc_bin_assign of libfgc_b200.so.
"""
import ctypes
from typing import Optional, Tuple

import torch

from .. import _cabi


def bin_by_coordinates(coordinates: torch.Tensor, row_splits: torch.Tensor,
                       bin_width: Optional[torch.Tensor] = None,
                       n_bins: Optional[torch.Tensor] = None, calc_n_per_bin: bool = True,
                       pre_normalized: bool = False, name: str = ""
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Assign bins to coordinates (TorchScript-compatible front of ``fgc_b200::bin_by_coordinates``;
    arguments, results and errors as documented at bin_by_coordinates_impl)."""
    if bin_width is None and n_bins is None:
        raise ValueError("Either bin_width or n_bins must be provided.")
    if torch.jit.is_scripting():
        return torch.ops.fgc_b200.bin_by_coordinates(coordinates, row_splits, bin_width, n_bins,
                                                     calc_n_per_bin, pre_normalized)
    else:
        if torch.jit.is_tracing():
            return torch.ops.fgc_b200.bin_by_coordinates(coordinates, row_splits, bin_width, n_bins,
                                                         calc_n_per_bin, pre_normalized)
        return bin_by_coordinates_impl(coordinates, row_splits, bin_width, n_bins, calc_n_per_bin,
                                       pre_normalized, name)


def bin_by_coordinates_impl(coordinates: torch.Tensor, row_splits: torch.Tensor,
                            bin_width: Optional[torch.Tensor] = None,
                            n_bins: Optional[torch.Tensor] = None, calc_n_per_bin: bool = True,
                            pre_normalized: bool = False, name: str = ""
                            ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Assign bins to coordinates.

    Args:
        coordinates: [n_vert, n_coords] (any float dtype, converted to float32).
        row_splits: ragged-tensor row splits (any integer dtype).
        bin_width: [1] uniform bin width; used if ``n_bins`` is not given.
        n_bins: scalar or [n_coords] number of bins; used if ``bin_width`` is not given.
        calc_n_per_bin: also return the histogram.
        pre_normalized: coordinates already start at 0 in every dimension.
        name: only used in error messages.

    Returns:
        (bin_indices [n_vert, n_coords+1] int64 = [row split, bin per dimension],
         flat_bin_indices [n_vert] int64, n_bins [n_coords] int64, bin_width [1] float32,
         n_per_bin [prod(n_bins)*(len(row_splits)-1)] int64).

    Raises ValueError for non-finite coordinates, a missing bin_width/n_bins pair,
    n_bins <= 0 or bin_width <= 0, as the reference does.
    """
    _cabi.require_cuda(coordinates, "coordinates")
    dev = coordinates.device
    if coordinates.dim() != 2:
        raise ValueError("coordinates must be [n_vert, n_coords]")
    n_vert, n_coords = coordinates.shape
    if n_coords < 1 or n_coords > _cabi.FGC_MAX_BIN_DIMS:
        raise ValueError("bin_by_coordinates supports 1..%d coordinate dimensions, got %d"
                         % (_cabi.FGC_MAX_BIN_DIMS, n_coords))
    if bin_width is None and n_bins is None:
        raise ValueError("Either bin_width or n_bins must be provided.")

    coords = coordinates.detach().to(dtype=torch.float32).contiguous()
    rs = row_splits.to(device=dev, dtype=torch.int64).contiguous()
    bw = None
    if bin_width is not None:
        if not torch.is_tensor(bin_width):
            bin_width = torch.tensor([bin_width], dtype=torch.float32)
        bw = bin_width.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
    nb = None
    if n_bins is not None:
        if not torch.is_tensor(n_bins):
            n_bins = torch.tensor(n_bins, dtype=torch.int64)
        nb = n_bins.to(device=dev, dtype=torch.int64).reshape(-1).contiguous()
        if nb.numel() not in (1, n_coords):
            raise ValueError("n_bins must be a scalar or have one entry per coordinate dimension")

    with torch.cuda.device(dev):
        stream = _cabi.current_stream(dev)
        params = torch.empty(256, dtype=torch.uint8, device=dev)
        _cabi.check(_cabi.lib.fgc_bin_prepare(
            _cabi.ptr(coords), n_vert, n_coords, int(bool(pre_normalized)), _cabi.ptr(bw),
            _cabi.ptr(nb), 0 if nb is None else nb.numel(), _cabi.ptr(params), stream),
            "fgc_bin_prepare")
        host = _cabi.BinParams.from_buffer_copy(params.cpu().numpy().tobytes())
        if host.status & _cabi.STATUS_NONFINITE:
            raise ValueError(f"BinByCoordinates: input coordinates {name} contain non-finite values")
        if host.status & _cabi.STATUS_BAD_DMAX:
            raise ValueError("BinByCoordinates: dmax_coords must be greater than zero.")
        if host.status & _cabi.STATUS_BAD_NBINS:
            raise ValueError("BinByCoordinates: n_bins must be greater than zero.")
        if host.status & _cabi.STATUS_BAD_BINWIDTH:
            raise ValueError("BinByCoordinates: bin_width must be greater than zero.")
        nb_list = [int(host.n_bins[c]) for c in range(n_coords)]
        n_total = 1
        for b in nb_list:
            n_total *= b
        n_total *= max(int(rs.numel()) - 1, 0)

        bin_indices = torch.zeros((n_vert, n_coords + 1), dtype=torch.int64, device=dev)
        flat = torch.zeros((n_vert,), dtype=torch.int64, device=dev)
        n_per_bin = torch.zeros((n_total,), dtype=torch.int64, device=dev)
        _cabi.check(_cabi.lib.fgc_bin_assign(
            _cabi.ptr(coords), n_vert, n_coords, _cabi.ptr(rs), rs.numel(), _cabi.ptr(params),
            int(bool(calc_n_per_bin)), n_total, _cabi.ptr(bin_indices), _cabi.ptr(flat),
            _cabi.ptr(n_per_bin), stream), "fgc_bin_assign")
    n_bins_out = torch.tensor(nb_list, dtype=torch.int64, device=dev)
    bin_width_out = torch.tensor([host.bin_width], dtype=torch.float32, device=dev)
    return bin_indices, flat, n_bins_out, bin_width_out, n_per_bin
