"""Draft-vocabulary construction from token frequencies.

The draft predicts over the ``draft_vocab_size`` most frequent verifier tokens.
``t2d`` is a bool mask over the verifier vocabulary marking the kept ids; ``d2t``
stores, for draft id ``i``, the *offset* ``target_id - i`` (so ``target = i +
d2t[i]``), which is the convention vLLM's EAGLE-3 loader expects.  Ties in
frequency are broken by the lower token id.  Parity:
src/speculators/train/vocab_mapping.py:17-125.
"""

from __future__ import annotations

import os
from collections import Counter

import torch

from speculators_b200.layer_config import read_config_json, unwrap_text_config

__all__ = [
    "build_vocab_mappings_from_distribution", "combine_token_frequency_distributions",
    "get_target_vocab_size", "save_token_frequency_distribution", "token_frequency_from_ids",
]


def token_frequency_from_ids(input_ids, loss_mask=None) -> dict[int, int]:
    """Counts of the token ids that take part in the loss."""
    ids = torch.as_tensor(input_ids).reshape(-1)
    if loss_mask is not None:
        ids = ids[torch.as_tensor(loss_mask).reshape(-1).bool()]
    values, counts = torch.unique(ids, return_counts=True)
    return dict(zip(values.tolist(), counts.tolist()))


def save_token_frequency_distribution(dataset, output_path: str) -> dict[int, int]:
    """Accumulate loss-masked token counts over ``dataset`` rows (``input_ids``,
    ``loss_mask``) and save them as ``token_freq.pt``."""
    total: Counter = Counter()
    for row in dataset:
        total.update(token_frequency_from_ids(row["input_ids"], row.get("loss_mask")))
    os.makedirs(os.path.dirname(os.path.abspath(output_path)), exist_ok=True)
    torch.save(dict(total), output_path)
    return dict(total)


def combine_token_frequency_distributions(distributions) -> dict[int, int]:
    total: Counter = Counter()
    for d in distributions:
        total.update(d)
    return dict(total)


def build_vocab_mappings_from_distribution(token_freq_dict: dict[int, int], draft_vocab_size: int, target_vocab_size: int):
    """-> ``(d2t int64[draft], t2d bool[target])``."""
    if draft_vocab_size > target_vocab_size:
        raise ValueError(f"draft_vocab_size ({draft_vocab_size}) exceeds target_vocab_size ({target_vocab_size})")
    freq = torch.zeros(target_vocab_size, dtype=torch.float64)
    for tok, count in token_freq_dict.items():
        if 0 <= int(tok) < target_vocab_size:
            freq[int(tok)] = float(count)
    # stable sort on descending frequency keeps lower ids first among ties
    order = torch.sort(-freq, stable=True).indices[:draft_vocab_size]
    kept = torch.sort(order).values
    d2t = kept - torch.arange(draft_vocab_size)
    t2d = torch.zeros(target_vocab_size, dtype=torch.bool)
    t2d[kept] = True
    return d2t.to(torch.long), t2d


def get_target_vocab_size(target_vocab_size: int | None, verifier_name_or_path: str | None) -> int:
    if target_vocab_size is not None:
        return int(target_vocab_size)
    if verifier_name_or_path is None:
        raise ValueError("either target_vocab_size or verifier_name_or_path is required")
    return int(unwrap_text_config(read_config_json(verifier_name_or_path))["vocab_size"])
