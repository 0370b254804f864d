"""Attention entry points shared by the model families.

The reference registers a flex-attention forward with HF and builds dense 0/-inf masks
for its eager / SDPA fallbacks (src/speculators/models/attention.py:20-108).  Here every
family describes its mask as an ``AttnSpec`` and calls ``masked_attention`` (sm_100a
kernels on CUDA, dense fp32 formulation elsewhere); ``create_float_mask`` gives the dense
additive mask of a spec for code that wants to feed another attention implementation.
"""

from __future__ import annotations

import torch

from speculators_b200.ops.attention import AttnSpec, masked_attention, masked_attention_reference

__all__ = ["ALL_ATTENTION_FUNCTIONS", "AttnSpec", "create_float_mask", "masked_attention", "masked_attention_reference"]


def create_float_mask(spec: AttnSpec, n_ctx: int, n_extra: int = 0, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Additive mask ``[Tq, n_ctx + n_extra]``: 0 where attention is allowed, ``-inf``
    elsewhere (rows without any allowed key are all ``-inf``; callers that softmax over
    such rows must handle them, ``masked_attention`` returns zeros there)."""
    allowed = spec.dense(n_ctx, n_extra)
    return torch.zeros(allowed.shape, dtype=dtype, device=allowed.device).masked_fill(~allowed, float("-inf"))


class _AttentionFunctions(dict):
    """Name -> attention function ``fn(q, k_ctx, v_ctx, spec, k_ext=None, v_ext=None,
    scale=None)`` (the role of the reference's ``ALL_ATTENTION_FUNCTIONS`` registry,
    src/speculators/models/attention.py:106-108, with this package's call signature):
    ``"masked"`` runs the sm_100a kernels (tcgen05 at head dim 128) with the dense fp32
    formulation as its CPU path, ``"reference"`` is that dense formulation everywhere."""

    def register(self, name: str, fn) -> None:  # noqa: ANN001
        self[name] = fn


ALL_ATTENTION_FUNCTIONS = _AttentionFunctions(masked=masked_attention, reference=masked_attention_reference)
