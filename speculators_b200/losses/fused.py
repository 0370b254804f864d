"""Fused (single-kernel) losses: same signatures as ``eager``, no ``[T, V]``
intermediate in forward or saved for backward.  CUDA inputs run the sm_100a
row-loss kernels (``ops/csrc/loss.cu``); the reference gets the same effect from
Triton programs (src/speculators/losses/fused.py).  On CPU the functions fall
through to the dense formulation so callers never branch on device.
"""

from __future__ import annotations

import torch

from speculators_b200.ops import fused_row_loss

_NLA_EPS = 1e-5

__all__ = [
    "fused_ce_loss",
    "fused_js_div_loss",
    "fused_kl_div_loss",
    "fused_lk_hybrid_loss",
    "fused_nla_loss",
    "fused_reverse_kl_div_loss",
    "fused_tv_loss",
]


def _rows(op: str, logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    lead = logits.shape[:-1]
    V = logits.shape[-1]
    lg = logits.reshape(-1, V) if logits.dim() != 2 else logits
    tg = targets.reshape(-1, V) if targets.dim() != 2 else targets
    loss, _, _ = fused_row_loss(op, lg, tg)
    return loss.reshape(lead)


def fused_kl_div_loss(logits, targets):
    return _rows("kl_div", logits, targets)


def fused_reverse_kl_div_loss(logits, targets):
    return _rows("rkl", logits, targets)


def fused_js_div_loss(logits, targets):
    return _rows("jsd", logits, targets)


def fused_ce_loss(logits, targets):
    return _rows("ce", logits, targets)


def fused_tv_loss(logits, targets):
    return _rows("tv", logits, targets)


def fused_nla_loss(logits, targets):
    alpha = 1.0 - fused_tv_loss(logits, targets)
    return -torch.log(alpha.clamp_min(_NLA_EPS))


def fused_lk_hybrid_loss(logits, targets, eta: float = 3.0):
    tv = fused_tv_loss(logits, targets)
    lam = torch.exp(-eta * (1.0 - tv).detach())
    return lam * fused_kl_div_loss(logits, targets) + (1.0 - lam) * tv
