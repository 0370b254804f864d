"""DSpark heads: a low-rank Markov correction of the draft logits and a per-slot acceptance
predictor (parameter names and math of src/speculators/models/dspark/model_definitions.py:12-91,
so checkpoints are interchangeable).

Markov head.  Slot ``k`` of a block gets the bias ``W2 . f_k`` with ``f_k`` a rank-``r`` feature
of the previous block token ``e_k = W1[prev_k]``:

* ``vanilla``  ``f_k = e_k``
* ``gated``    ``f_k = sigmoid(G [h_k; e_k] + g) * e_k``
* ``rnn``      ``z_k = J [s_{k-1}; e_k; h_k] + j`` split into (gate, candidate, emit);
               ``s_k = sig(gate) s_{k-1} + (1 - sig(gate)) tanh(candidate)``, ``f_k = tanh(emit)``

Everything that does not depend on the recurrent state is computed for all ``N * B`` rows at
once on the package's GEMM: the ``[e; h]`` part of ``J`` is one product over every slot (only
the ``r x 3r`` state term stays in the loop over the block), and ``W2`` is applied once to the
stacked features, optionally with the backbone's logits as the GEMM's residual so that
"logits + bias" costs no extra pass.
"""

from __future__ import annotations

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.models.layers import Linear

__all__ = ["ConfidenceHead", "MarkovHead"]

_HEAD_TYPES = ("vanilla", "gated", "rnn")


class MarkovHead(nn.Module):
    def __init__(self, *, verifier_vocab_size: int, draft_vocab_size: int, markov_rank: int, hidden_size: int, head_type: str = "vanilla"):
        super().__init__()
        if markov_rank <= 0:
            raise ValueError(f"markov_rank must be > 0, got {markov_rank}")
        if head_type not in _HEAD_TYPES:
            raise ValueError(f"Unsupported markov_head_type: {head_type!r}")
        r = markov_rank
        self.head_type, self.markov_rank, self.hidden_size = head_type, r, hidden_size
        self.markov_w1 = nn.Embedding(verifier_vocab_size, r)
        self.markov_w2 = Linear(r, draft_vocab_size, bias=False)
        if head_type == "gated":
            self.gate_proj = Linear(hidden_size + r, r, bias=True)  # input order [h; e]
        elif head_type == "rnn":
            self.joint_proj = Linear(2 * r + hidden_size, 3 * r, bias=True)  # input order [s; e; h]

    def prev_embeddings(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.markov_w1(token_ids.long())

    # ------------------------------------------------------------------ features f_k
    def features(self, prev_emb: torch.Tensor, hidden_states: torch.Tensor | None) -> torch.Tensor:
        """``[N, B, r]`` embeddings (+ ``[N, B, H]`` states) -> ``[N, B, r]`` features."""
        e = prev_emb.to(self.markov_w2.weight.dtype)
        if self.head_type == "vanilla":
            return e
        h = hidden_states.to(e.dtype)
        if self.head_type == "gated":
            return torch.sigmoid(self.gate_proj(torch.cat([h, e], dim=-1))) * e
        return self._recurrent_features(e, h)

    def _recurrent_features(self, e: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        n, width, r = e.shape
        w, b = self.joint_proj.weight, self.joint_proj.bias
        # state-independent part for every slot at once: J[:, r:] [e; h] + j
        fixed = ops.linear(torch.cat([e, h], dim=-1).reshape(n * width, -1), w[:, r:], b).view(n, width, 3 * r)
        w_state = w[:, :r]
        state = e.new_zeros(n, r)
        emitted = []
        for k in range(width):
            z = fixed[:, k] + state @ w_state.t() if k else fixed[:, 0]
            gate, candidate, emit = z.split(r, dim=-1)
            gate = torch.sigmoid(gate)
            state = gate * state + (1.0 - gate) * torch.tanh(candidate)
            emitted.append(torch.tanh(emit))
        return torch.stack(emitted, dim=1)

    # ------------------------------------------------------------------ bias = W2 f
    def add_to_logits(self, logits2d: torch.Tensor, feats: torch.Tensor) -> torch.Tensor:
        """``logits2d + W2 f`` for ``[N * B, V]`` logits: one GEMM with the logits as its residual."""
        return self.markov_w2(feats.reshape(logits2d.shape[0], -1), residual=logits2d)

    def block_bias(self, *, prev_token_ids: torch.Tensor, hidden_states: torch.Tensor | None, prev_emb: torch.Tensor | None = None) -> torch.Tensor:
        """``[N, B]`` ids (and ``[N, B, H]`` states) -> ``[N, B, draft_vocab]`` bias."""
        if prev_emb is None:
            prev_emb = self.prev_embeddings(prev_token_ids)
        feats = self.features(prev_emb, hidden_states)
        n, width, _ = feats.shape
        return self.markov_w2(feats.reshape(n * width, -1)).view(n, width, -1)


class ConfidenceHead(nn.Module):
    """One linear unit per slot: the logit of the probability that the slot's token is accepted."""

    def __init__(self, input_dim: int):
        super().__init__()
        self.proj = Linear(input_dim, 1, bias=True)

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        # a single output unit is a row-wise dot product: done in fp32 as multiply + reduce
        w = self.proj.weight.reshape(-1).float()
        return (features.float() * w).sum(dim=-1).add(self.proj.bias.float()).to(features.dtype)
