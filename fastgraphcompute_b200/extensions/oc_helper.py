"""select_with_default -- the one function of fastgraphcompute.extensions.oc_helper that
the GravNet path uses (extensions/oc_helper.py:232-271).  Thin tensor code: the
GravNet layer itself never calls it, its fused kernel applies the same rule
(-1 -> default) without building the [V, K, F] tensor."""
import torch


def select_with_default(idx: torch.Tensor, feat: torch.Tensor, default_value: float) -> torch.Tensor:
    """out[v, k, :] = feat[idx[v, k], :], or ``default_value`` where idx[v, k] == -1.

    idx: [V, K] integer tensor; feat: [V, F]; returns [V, K, F] with feat's dtype.
    """
    idx = idx.long()
    valid = (idx != -1).unsqueeze(-1)
    gathered = feat[idx.clamp(min=0)]
    return torch.where(valid, gathered, torch.full((), default_value, dtype=feat.dtype,
                                                   device=feat.device))
