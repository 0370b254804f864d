"""Seeded synthetic training batches (no dataset, no tokenizer, no network).

Shapes follow what ``CollateFn`` hands the trainer after ``shift_batch``
(``[1, T, ...]`` with one packed row, src/speculators/train/data.py:344-393;
the reference's own benchmark builds the same dict in
scripts/benchmark.py:187-210).  Token ids are uniform, the loss mask is drawn per
span (each span fully on with probability ``p``), documents are contiguous runs,
and hidden states come either from a ``RandomVerifier`` forward or, when
``verifier`` is None, from a unit normal.
"""

from __future__ import annotations

import torch

__all__ = ["SyntheticLoader", "make_eagle3_batch", "span_bernoulli_mask"]


def span_bernoulli_mask(T: int, p: float, span: int, gen: torch.Generator) -> torch.Tensor:
    n_spans = (T + span - 1) // span
    on = torch.rand(n_spans, generator=gen) < p
    return on.repeat_interleave(span)[:T]


def make_eagle3_batch(
    total_seq_len: int, hidden_size: int, num_aux: int, vocab_size: int, *, seed: int = 0, mask_p: float = 0.6,
    mask_span: int = 64, num_documents: int = 1, pad_tokens: int = 0, dtype=torch.bfloat16, verifier=None,
    layer_ids: list[int] | None = None, pin: bool = False,
) -> dict[str, torch.Tensor]:
    """One post-collate EAGLE-3 / P-EAGLE batch on the host."""
    gen = torch.Generator().manual_seed(seed)
    T = total_seq_len
    ids = torch.randint(0, vocab_size, (T,), generator=gen)
    mask = span_bernoulli_mask(T, mask_p, mask_span, gen)
    real = T - pad_tokens
    bounds = torch.linspace(0, real, num_documents + 1).long()
    doc = torch.full((T,), -1, dtype=torch.long)
    pos = torch.zeros(T, dtype=torch.long)
    for d in range(num_documents):
        a, b = int(bounds[d]), int(bounds[d + 1])
        doc[a:b] = d
        pos[a:b] = torch.arange(1, b - a + 1)
    mask = mask & (doc != -1)
    if verifier is not None:
        out = verifier.forward(ids, layer_ids, document_ids=doc, position_ids=pos)
        hs = out["hidden_states"].to("cpu", dtype)
        last = out["verifier_last_hidden_states"].to("cpu", dtype)
    else:
        hs = torch.randn(T, num_aux * hidden_size, generator=gen).to(dtype)
        last = torch.randn(T, hidden_size, generator=gen).to(dtype)
    batch = {
        "hidden_states": hs.unsqueeze(0), "input_ids": ids.unsqueeze(0), "verifier_last_hidden_states": last.unsqueeze(0),
        "loss_mask": mask.unsqueeze(0), "position_ids": pos.unsqueeze(0), "document_ids": doc.unsqueeze(0),
    }
    if pin and torch.cuda.is_available():
        batch = {k: v.contiguous().pin_memory() for k, v in batch.items()}
    return batch


class SyntheticLoader:
    """Loader-shaped wrapper (``__len__``, ``__iter__``, ``batch_sampler.set_epoch``)
    that cycles through a fixed list of host batches."""

    class _Sampler:
        def set_epoch(self, _epoch: int) -> None:
            pass

    def __init__(self, batches: list[dict] | dict, num_steps: int):
        if isinstance(batches, dict):  # one batch, repeated
            batches = [batches]
        self.batches, self.num_steps = batches, num_steps
        self.batch_sampler = self._Sampler()

    def __len__(self) -> int:
        return self.num_steps

    def __iter__(self):
        for i in range(self.num_steps):
            yield self.batches[i % len(self.batches)]
