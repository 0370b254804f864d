"""DSpark draft model = DFlash backbone + Markov head + confidence head
(behaviour of src/speculators/models/dspark/core.py:27-212).

The backbone yields, for ``N`` anchored blocks of ``B`` slots, hidden states and logits
``[N * B, .]``.  The Markov head corrects the logits of slot ``k`` with a low-rank function of
the block's previous token (added in the epilogue of the head's own GEMM); the confidence head
reads ``[h_k; e_k]`` and predicts the slot's acceptance probability.  Shapes are fixed by
``max_anchors`` and the block size, so the whole step can be captured in a CUDA graph.
"""

from __future__ import annotations

from typing import ClassVar

import torch

from speculators_b200.losses import LossConfig, kl_div_loss, resolve_loss_config, tv_loss
from speculators_b200.model import SpeculatorModel
from speculators_b200.models.dflash.core import DFlashDraftModel
from speculators_b200.models.dspark.config import DSparkSpeculatorConfig
from speculators_b200.models.dspark.metrics import compute_metrics
from speculators_b200.models.dspark.model_definitions import ConfidenceHead, MarkovHead

__all__ = ["DSparkDraftModel"]

# train / validation call keywords and the command-line names they come from (with defaults)
_CALL_KWARGS = {
    "gamma": ("dflash_decay_gamma", 4.0),
    "max_anchors": ("max_anchors", 3072),
    "confidence_head_alpha": ("confidence_head_alpha", 1.0),
    "per_position_loss_weight": ("per_position_loss_weight", "fixed-exp-decay"),
    "dpace_alpha": ("dpace_alpha", 0.5),
}


def _or_default(value, default):
    return default if value is None else value


@SpeculatorModel.register("dspark")
class DSparkDraftModel(DFlashDraftModel):
    config_class: ClassVar[type[DSparkSpeculatorConfig]] = DSparkSpeculatorConfig

    def __init__(self, config: DSparkSpeculatorConfig):
        super().__init__(config=config)
        width = config.transformer_layer_config.hidden_size
        rank = config.markov_rank
        self.markov_head = self.confidence_head = None
        if rank > 0:
            self.markov_head = MarkovHead(
                verifier_vocab_size=self.verifier_vocab_size, draft_vocab_size=self.draft_vocab_size, markov_rank=rank,
                hidden_size=width, head_type=config.markov_head_type,
            )
        if config.enable_confidence_head:
            sees_markov = bool(config.confidence_head_with_markov)
            if sees_markov and self.markov_head is None:
                raise ValueError("confidence_head_with_markov=True requires markov_rank > 0.")
            self.confidence_head = ConfidenceHead(width + (rank if sees_markov else 0))

    # ------------------------------------------------------------------ construction from the CLI
    @classmethod
    def from_training_args(cls, verifier_config, t2d=None, d2t=None, **kwargs) -> "DSparkDraftModel":
        base = cls._build_base_config_kwargs("dspark", verifier_config, **kwargs)
        model = cls(config=DSparkSpeculatorConfig(
            **base,
            markov_rank=kwargs.get("markov_rank", 256),
            markov_head_type=kwargs.get("markov_head_type", "vanilla"),
            enable_confidence_head=_or_default(kwargs.get("enable_confidence_head"), True),
            confidence_head_with_markov=_or_default(kwargs.get("confidence_head_with_markov"), True),
        ))
        model.load_vocab_mappings(t2d, d2t)
        model.load_verifier_weights()
        return model

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        implementation = kwargs.get("loss_implementation", "fused")
        call = {name: kwargs.get(flag, default) for name, (flag, default) in _CALL_KWARGS.items()}
        call["loss_config"] = resolve_loss_config(kwargs["loss_fn"], implementation)
        call["tv_loss_fn"] = resolve_loss_config("tv", implementation)["tv"][0]
        return dict(call), dict(call)

    # ------------------------------------------------------------------ heads
    def _previous_tokens(self, input_ids: torch.Tensor, block_index: torch.Tensor, blocks: int) -> torch.Tensor:
        """``[N, B]`` token that precedes each slot's prediction: the slot's own token when slot 0
        predicts (sample_from_anchor), else the token one slot to the left (the anchor for slot 0)."""
        flat = input_ids.reshape(-1)
        tokens = flat[block_index % flat.shape[0]].view(blocks, self.block_size)
        if self.config.sample_from_anchor:
            return tokens
        return torch.cat([tokens[:, :1], tokens[:, :-1]], dim=1)

    def _apply_heads(self, hidden: torch.Tensor, logits: torch.Tensor, prev_ids: torch.Tensor):
        """``hidden`` / ``logits`` ``[1, N * B, .]`` -> (corrected logits ``[1, N * B, V]``, confidence logits ``[1, N * B]`` or None)."""
        blocks, width = prev_ids.shape
        states = hidden.view(blocks, width, -1)
        emb = None
        if self.markov_head is not None:
            emb = self.markov_head.prev_embeddings(prev_ids)
            feats = self.markov_head.features(emb, states)
            logits = self.markov_head.add_to_logits(logits.reshape(blocks * width, -1), feats).unsqueeze(0)
        confidence = None
        if self.confidence_head is not None:
            seen = states
            if self.config.confidence_head_with_markov and emb is not None:
                seen = torch.cat([states, emb.to(states.dtype)], dim=-1)
            confidence = self.confidence_head(seen).reshape(1, blocks * width)
        return logits, confidence

    def forward(self, hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids=None,
                loss_config: LossConfig | None = None, tv_loss_fn=tv_loss, gamma: float = 4.0, max_anchors: int = 3072,
                confidence_head_alpha: float = 1.0, per_position_loss_weight: str = "fixed-exp-decay", dpace_alpha: float = 0.5, **kwargs):
        hidden, logits, targets, slot_mask, block_index = self._backbone_forward(
            hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids, max_anchors=max_anchors
        )
        logits, confidence = self._apply_heads(hidden, logits, self._previous_tokens(input_ids, block_index, max_anchors))
        loss, metrics = compute_metrics(
            logits, targets, confidence, slot_mask, self.block_size, loss_config=loss_config or {"kl_div": (kl_div_loss, 1.0)},
            tv_loss_fn=tv_loss_fn, gamma=gamma, confidence_head_alpha=confidence_head_alpha,
            per_position_loss_weight=per_position_loss_weight, dpace_alpha=dpace_alpha,
            sample_from_anchor=self.config.sample_from_anchor,
        )
        return None, loss, metrics
