"""Dense PyTorch losses between draft logits and verifier logits.

Each function maps ``logits, targets`` of shape ``[B, T, V]`` to a per-position
fp32 loss ``[B, T]``.  They materialise ``[T, V]`` fp32 intermediates and exist as
the numerical oracle for the fused kernels and for CPU runs.  Definitions follow
src/speculators/losses/eager.py:11-213 (KL(p||q), reverse KL, Jensen-Shannon, CE
against ``argmax(targets)``, total variation ``1 - sum min(p, q)``, negative log
acceptance ``-log max(alpha, 1e-5)`` and the LK hybrid
``lam*KL + (1-lam)*TV`` with ``lam = exp(-eta * stopgrad(alpha))``).
"""

from __future__ import annotations

import torch

from speculators_b200.ops import _row_loss_ref

_NLA_EPS = 1e-5

__all__ = [
    "ce_loss",
    "js_div_loss",
    "kl_div_loss",
    "lk_hybrid_loss",
    "neg_log_acceptance_loss",
    "reverse_kl_div_loss",
    "tv_loss",
]


def _rows(op: str, logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    lead = logits.shape[:-1]
    V = logits.shape[-1]
    out = _row_loss_ref(op, logits.reshape(-1, V), targets.reshape(-1, V))
    return out.reshape(lead)


def kl_div_loss(logits, targets):
    return _rows("kl_div", logits, targets)


def reverse_kl_div_loss(logits, targets):
    return _rows("rkl", logits, targets)


def js_div_loss(logits, targets):
    return _rows("jsd", logits, targets)


def ce_loss(logits, targets):
    return _rows("ce", logits, targets)


def tv_loss(logits, targets):
    return _rows("tv", logits, targets)


def neg_log_acceptance_loss(logits, targets):
    alpha = 1.0 - tv_loss(logits, targets)
    return -torch.log(alpha.clamp_min(_NLA_EPS))


def lk_hybrid_loss(logits, targets, eta: float = 3.0):
    tv = tv_loss(logits, targets)
    lam = torch.exp(-eta * (1.0 - tv).detach())
    return lam * kl_div_loss(logits, targets) + (1.0 - lam) * tv
