"""Per-sample alignment for EAGLE-3 / P-EAGLE: the draft at position ``t`` sees the
verifier's hidden state of token ``t-1`` together with token ``t`` itself, and is
trained against the verifier's output at ``t``.  Dropping the first token /
last hidden state implements that pairing, and ``position_ids`` consequently
start at 1 (src/speculators/models/eagle3/data.py:28-44)."""

from __future__ import annotations

import torch

__all__ = ["shift_batch"]


def shift_batch(batch: dict) -> dict:
    return {
        "input_ids": batch["input_ids"][1:],
        "hidden_states": batch["hidden_states"][:-1],
        "verifier_last_hidden_states": batch["verifier_last_hidden_states"][1:],
        "loss_mask": batch["loss_mask"][1:],
        "lengths": torch.clamp(batch["lengths"] - 1, min=0),  # empty fallback sample stays at 0
        "position_ids": batch["position_ids"][1:],
    }
