"""Row-level evaluation of a ``LossConfig`` with target shift and argmax by-products.

``rowwise_terms`` is what the algorithm metrics call.  For every configured term
whose function is one of the registered losses it runs the shift-aware kernel
(``ops.fused_row_loss``) or, for the eager implementation, the dense formula on
slice views; unknown callables are applied to ``[1, rows, V]`` slice views.
"""

from __future__ import annotations

import torch

from speculators_b200.losses import eager, fused
from speculators_b200.losses.utils import LossConfig, loss_name_of
from speculators_b200.ops import fused_row_loss

__all__ = ["rowwise_terms"]

_PRIMITIVES = ("kl_div", "rkl", "jsd", "ce", "tv")
_NLA_EPS = 1e-5


def _is_fused(fn) -> bool:
    return getattr(fn, "__module__", "") == fused.__name__


def rowwise_terms(loss_config: LossConfig, logits2d, targets2d, shift: int, rows: int, active=None):
    """-> ``({name: loss[rows]}, argmax_logits[rows], argmax_targets[rows])``."""
    out: dict[str, torch.Tensor] = {}
    am_d = am_t = None

    def prim(op: str):
        nonlocal am_d, am_t
        loss, a, b = fused_row_loss(op, logits2d, targets2d, shift=shift, rows=rows, active=active)
        if am_d is None:
            am_d, am_t = a, b
        return loss

    for name, (fn, _w) in loss_config.items():
        known = loss_name_of(fn)
        if known is not None and _is_fused(fn):
            if known in _PRIMITIVES:
                out[name] = prim(known)
            elif known == "nla":
                out[name] = -torch.log((1.0 - prim("tv")).clamp_min(_NLA_EPS))
            else:  # lk_hybrid
                tv = prim("tv")
                lam = torch.exp(-3.0 * (1.0 - tv).detach())
                out[name] = lam * prim("kl_div") + (1.0 - lam) * tv
        else:
            lg = logits2d[:rows].unsqueeze(0)
            tg = targets2d[shift : shift + rows].unsqueeze(0)
            out[name] = fn(lg, tg).reshape(rows)
    if am_d is None:
        am_d = logits2d[:rows].argmax(-1)
        am_t = targets2d[shift : shift + rows].argmax(-1)
    return out, am_d, am_t
