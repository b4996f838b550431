"""index_replacer -- drop-in for fastgraphcompute.extensions.index_replacer
(extensions/index_replacer.py:40-59)."""
import torch

from .. import _cabi



def index_replacer_eager(to_be_replaced: torch.Tensor, replacements: torch.Tensor) -> torch.Tensor:
    """fgc_index_replacer on prepared tensors (what the dispatcher op fgc_b200::index_replacer runs)."""
    _cabi.require_cuda(to_be_replaced, "to_be_replaced")
    src = to_be_replaced.contiguous()
    rep = replacements.contiguous()
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        _cabi.check(_cabi.lib.fgc_index_replacer(
            _cabi.ptr(src), src.numel(), _cabi.ptr(rep), rep.shape[0] if rep.dim() else 0,
            _cabi.ptr(out), _cabi.current_stream(src.device)), "fgc_index_replacer")
    return out


def index_replacer(to_be_replaced: torch.Tensor, replacements: torch.Tensor) -> torch.Tensor:
    """Replace every non-negative entry v of ``to_be_replaced`` by ``replacements[v]``.

    Negative entries are kept.  Both tensors must be int64 and on the same device;
    the result has the shape and dtype of ``to_be_replaced``.
    """
    if to_be_replaced.device != replacements.device:
        raise AssertionError("Tensors must be on the same device.")
    if to_be_replaced.dtype != torch.int64 or replacements.dtype != torch.int64:
        raise AssertionError("Tensors must be int64 type.")
    if torch.jit.is_scripting():
        return torch.ops.fgc_b200.index_replacer(to_be_replaced, replacements)
    else:
        if torch.jit.is_tracing():
            return torch.ops.fgc_b200.index_replacer(to_be_replaced, replacements)
        return index_replacer_eager(to_be_replaced, replacements)
