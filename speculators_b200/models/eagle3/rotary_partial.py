"""Partial rotary embedding (neox layout): rotate the first ``rotary_dim`` channels of
every head, pass the rest through.

The reference needs a monkey-patch of HF's ``apply_rotary_pos_emb`` to get this for Llama /
Qwen3 blocks (src/speculators/models/eagle3/rotary_partial.py:27-106).  Here partial
rotation is a parameter of the attention block itself (``Attention.rot``, taken from
``partial_rotary_factor`` / ``rotary_dim``) and of the rotary kernel, so
``install_partial_neox_rotary`` has nothing to patch; it is kept as a no-op so callers
written against the reference's API keep working.  ``partial_neox_apply_rotary_pos_emb``
is the tensor-level function with the reference's signature (used by tests as the oracle
of the kernel's partial mode).
"""

from __future__ import annotations

import torch

__all__ = ["install_partial_neox_rotary", "partial_neox_apply_rotary_pos_emb", "uninstall_partial_neox_rotary"]


def _swap_halves(x: torch.Tensor) -> torch.Tensor:
    a, b = x.chunk(2, dim=-1)
    return torch.cat((-b, a), dim=-1)


def partial_neox_apply_rotary_pos_emb(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                                      unsqueeze_dim: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """``cos`` / ``sin`` of last dim ``rotary_dim <= head_dim``: channels ``[0, rotary_dim)``
    rotate, channels beyond stay as they are (``rotary_dim == head_dim`` is the usual full
    rotation)."""
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    rot = cos.shape[-1]
    if rot > q.shape[-1]:
        raise ValueError(f"cos last dim ({rot}) exceeds q last dim ({q.shape[-1]})")

    def apply(x: torch.Tensor) -> torch.Tensor:
        head, tail = x[..., :rot], x[..., rot:]
        turned = head * cos + _swap_halves(head) * sin
        return turned if tail.shape[-1] == 0 else torch.cat([turned, tail], dim=-1)

    return apply(q), apply(k)


def install_partial_neox_rotary() -> None:
    """No-op: the blocks of this package rotate partially by construction."""


def uninstall_partial_neox_rotary() -> None:
    """No-op counterpart of ``install_partial_neox_rotary``."""
