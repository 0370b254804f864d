"""DSpark heads (src/speculators/models/dspark/model_definitions.py:12-91).

``MarkovHead``: logit bias from the previous block token, factorised as
``W2(f(W1[prev]))`` with ``W1`` an embedding over the verifier vocabulary (rank
``r``) and ``W2: r -> draft vocab``.  ``f`` is the identity (``vanilla``), a
hidden-state-conditioned sigmoid gate (``gated``) or a small recurrent cell run
across the block (``rnn``).  ``ConfidenceHead``: one linear unit predicting the
per-position acceptance probability (as a logit).
"""

from __future__ import annotations

import torch
from torch import nn

__all__ = ["ConfidenceHead", "MarkovHead"]


class MarkovHead(nn.Module):
    def __init__(self, *, verifier_vocab_size: int, draft_vocab_size: int, markov_rank: int, hidden_size: int, head_type: str = "vanilla"):
        super().__init__()
        if markov_rank <= 0:
            raise ValueError(f"markov_rank must be > 0, got {markov_rank}")
        if head_type not in ("vanilla", "gated", "rnn"):
            raise ValueError(f"Unsupported markov_head_type: {head_type!r}")
        self.head_type, self.markov_rank = head_type, markov_rank
        self.markov_w1 = nn.Embedding(verifier_vocab_size, markov_rank)
        self.markov_w2 = nn.Linear(markov_rank, draft_vocab_size, bias=False)
        if head_type == "gated":
            self.gate_proj = nn.Linear(hidden_size + markov_rank, markov_rank)
        elif head_type == "rnn":
            self.joint_proj = nn.Linear(2 * markov_rank + hidden_size, 3 * markov_rank)

    def prev_embeddings(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.markov_w1(token_ids.long())

    def block_bias(self, *, prev_token_ids, hidden_states, prev_emb=None) -> torch.Tensor:
        """``[N, B]`` ids, ``[N, B, H]`` states -> ``[N, B, draft_vocab]`` bias."""
        if prev_emb is None:
            prev_emb = self.prev_embeddings(prev_token_ids)
        prev_emb = prev_emb.to(self.markov_w2.weight.dtype)
        if self.head_type == "vanilla":
            return self.markov_w2(prev_emb)
        hidden_states = hidden_states.to(prev_emb.dtype)
        if self.head_type == "gated":
            gate = torch.sigmoid(self.gate_proj(torch.cat([hidden_states, prev_emb], dim=-1)))
            return self.markov_w2(gate * prev_emb)
        blocks, width, _ = prev_emb.shape
        state = prev_emb.new_zeros(blocks, self.markov_rank)
        out = []
        for k in range(width):
            g, cand, emit = self.joint_proj(torch.cat([state, prev_emb[:, k], hidden_states[:, k]], dim=-1)).chunk(3, dim=-1)
            g = torch.sigmoid(g)
            state = g * state + (1.0 - g) * torch.tanh(cand)
            out.append(self.markov_w2(torch.tanh(emit)))
        return torch.stack(out, dim=1)


class ConfidenceHead(nn.Module):
    def __init__(self, input_dim: int):
        super().__init__()
        self.proj = nn.Linear(input_dim, 1)

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        return self.proj(features).squeeze(-1)
