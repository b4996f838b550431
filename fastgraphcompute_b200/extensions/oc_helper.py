"""Counterparts of fastgraphcompute.extensions.oc_helper (extensions/oc_helper.py of the
reference): ``select_with_default`` (lines 232-271) and ``oc_helper_matrices`` (128-230).

``select_with_default`` is the rule the GravNet layer applies to its neighbour indices
(-1 -> default); the layer's fused kernel applies it without building the [V, K, F] tensor,
this function builds it for callers that want it (the object-condensation loss).  On CUDA
tensors of 4- or 8-byte element types both functions run in libfgc_b200.so.
"""
import ctypes
import struct
from typing import Tuple

import torch

from .. import _cabi

_PACK = {torch.float32: "f", torch.float64: "d", torch.int32: "i", torch.int64: "q"}


def _select_with_default_tensor_code(idx, feat, default_value):
    idx = idx.long()
    valid = (idx != -1).unsqueeze(-1)
    gathered = feat[idx.clamp(min=0)]
    return torch.where(valid, gathered, torch.full((), default_value, dtype=feat.dtype, device=feat.device))


def _select_with_default_cuda(idx, feat, default_value):
    V, K = idx.shape
    F = feat.shape[1]
    out = torch.empty((V, K, F), dtype=feat.dtype, device=feat.device)
    fmt = _PACK[feat.dtype]
    word = struct.pack(fmt, default_value if fmt in "fd" else int(default_value))
    buf = ctypes.create_string_buffer(word, len(word))
    with torch.cuda.device(feat.device):
        _cabi.check(_cabi.lib.fgc_select_with_default(
            _cabi.ptr(idx), V * K, _cabi.ptr(feat), feat.shape[0], F, len(word),
            ctypes.cast(buf, ctypes.c_void_p), _cabi.ptr(out), _cabi.current_stream(feat.device)),
            "fgc_select_with_default")
    return out


class _SelectWithDefault(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, feat, default_value):
        ctx.save_for_backward(idx)
        ctx.n_rows = feat.shape[0]
        return _select_with_default_cuda(idx, feat, default_value)

    @staticmethod
    def backward(ctx, grad):
        (idx,) = ctx.saved_tensors
        flat = idx.reshape(-1)
        valid = flat >= 0
        g = grad.reshape(flat.shape[0], -1)
        out = torch.zeros((ctx.n_rows, g.shape[1]), dtype=grad.dtype, device=grad.device)
        out.index_add_(0, flat[valid], g[valid])
        return None, out, None


def select_with_default(idx: torch.Tensor, feat: torch.Tensor, default_value: float) -> torch.Tensor:
    """out[v, k, :] = feat[idx[v, k], :], or ``default_value`` where idx[v, k] == -1.

    idx: [V, K] integer tensor; feat: [N, F]; returns [V, K, F] with feat's dtype."""
    if (feat.is_cuda and idx.is_cuda and feat.dtype in _PACK and feat.dim() == 2 and idx.dim() == 2
            and not torch.jit.is_scripting() and not torch.jit.is_tracing()):
        idx = idx.to(torch.int64).contiguous()
        feat = feat.contiguous()
        if feat.requires_grad and torch.is_grad_enabled():
            return _SelectWithDefault.apply(idx, feat, default_value)
        return _select_with_default_cuda(idx, feat.detach(), default_value)
    return _select_with_default_tensor_code(idx, feat, default_value)


def oc_helper_matrices(truth_idxs: torch.Tensor, row_splits: torch.Tensor,
                       calc_m_not: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Index matrices of the object-condensation loss (oc_helper.py:128-230 of the reference).

    truth_idxs: [V] int64 truth index of every point (negative: no object); row_splits [R+1].
    Returns (M [K, n_max_points_per_object], M_not [K, n_max_points_per_row_split], both int64
    and padded with -1, objects_per_row_split [R]); an object never crosses a row split.  Row k
    of M lists the points of object k, row k of M_not all other points of its row split (only
    -1 when ``calc_m_not`` is False); use them with select_with_default.  Objects are ordered by
    (truth index, row split) -- the reference leaves the order open."""
    _cabi.require_cuda(truth_idxs, "truth_idxs")
    if truth_idxs.device != row_splits.device:
        raise RuntimeError("Both truth_idxs and row_splits must be on the same device")
    asso = truth_idxs.to(torch.int64).contiguous().reshape(-1)
    rs = row_splits.to(torch.int64).contiguous()
    n_vert, n_rs = asso.shape[0], rs.shape[0]
    dev = asso.device
    nbytes = _cabi.lib.fgc_oc_workspace_bytes(n_vert)
    if nbytes == 0:
        raise ValueError("oc_helper_matrices: unsupported problem size")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    per_split = torch.empty(max(n_rs - 1, 0), dtype=torch.int64, device=dev)
    status = ctypes.c_int32(0)
    sizes = (ctypes.c_int64 * 3)()
    with torch.cuda.device(dev):
        stream = _cabi.current_stream(dev)
        _cabi.check(_cabi.lib.fgc_oc_prepare(_cabi.ptr(asso), n_vert, _cabi.ptr(rs), n_rs, _cabi.ptr(ws), nbytes,
                                             _cabi.ptr(per_split), stream), "fgc_oc_prepare")
        _cabi.check(_cabi.lib.fgc_oc_read_sizes(_cabi.ptr(ws), ctypes.byref(status), sizes, stream),
                    "fgc_oc_read_sizes")
        if status.value & _cabi.STATUS_BAD_ROW_SPLITS:
            raise RuntimeError("oc_helper_matrices: row_splits must start at 0, end at len(truth_idxs) "
                               "and never decrease")
        n_unique, n_maxuq, n_maxrs = int(sizes[0]), int(sizes[1]), int(sizes[2])
        M = torch.empty((n_unique, n_maxuq), dtype=torch.int64, device=dev)
        if calc_m_not:
            M_not = torch.empty((n_unique, n_maxrs), dtype=torch.int64, device=dev)
        else:
            M_not = torch.full((n_unique, n_maxrs), -1, dtype=torch.int64, device=dev)
        _cabi.check(_cabi.lib.fgc_oc_fill(_cabi.ptr(ws), nbytes, n_vert, _cabi.ptr(rs), n_unique, n_maxuq, n_maxrs,
                                          _cabi.ptr(M), _cabi.ptr(M_not) if calc_m_not else None, stream),
                    "fgc_oc_fill")
    return M, M_not, per_split
