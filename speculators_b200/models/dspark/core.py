"""DSpark draft model: the DFlash backbone, then a Markov head that biases the
logits of slot ``k`` with the previous block token, and a confidence head that
predicts each slot's acceptance probability
(src/speculators/models/dspark/core.py:27-212)."""

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


@SpeculatorModel.register("dspark")
class DSparkDraftModel(DFlashDraftModel):
    config_class: ClassVar[type[DSparkSpeculatorConfig]] = DSparkSpeculatorConfig

    def __init__(self, config: DSparkSpeculatorConfig):
        super().__init__(config=config)
        H = config.transformer_layer_config.hidden_size
        self.markov_head = None
        if config.markov_rank > 0:
            self.markov_head = MarkovHead(
                verifier_vocab_size=self.verifier_vocab_size, draft_vocab_size=self.draft_vocab_size,
                markov_rank=config.markov_rank, hidden_size=H, head_type=config.markov_head_type,
            )
        self.confidence_head = None
        if config.enable_confidence_head:
            if config.confidence_head_with_markov and self.markov_head is None:
                raise ValueError("confidence_head_with_markov=True requires markov_rank > 0.")
            self.confidence_head = ConfidenceHead(H + (config.markov_rank if config.confidence_head_with_markov else 0))

    @classmethod
    def from_training_args(cls, verifier_config, t2d=None, d2t=None, **kwargs) -> "DSparkDraftModel":
        conf = kwargs.get("enable_confidence_head")
        with_markov = kwargs.get("confidence_head_with_markov")
        config = DSparkSpeculatorConfig(
            **cls._build_base_config_kwargs("dspark", verifier_config, **kwargs),
            markov_rank=kwargs.get("markov_rank", 256),
            markov_head_type=kwargs.get("markov_head_type", "vanilla"),
            enable_confidence_head=True if conf is None else conf,
            confidence_head_with_markov=True if with_markov is None else with_markov,
        )
        model = cls(config=config)
        model.load_vocab_mappings(t2d, d2t)
        model.load_verifier_weights()
        return model

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        impl = kwargs.get("loss_implementation", "fused")
        shared = {
            "loss_config": resolve_loss_config(kwargs["loss_fn"], impl),
            "tv_loss_fn": resolve_loss_config("tv", impl)["tv"][0],
            "gamma": kwargs.get("dflash_decay_gamma", 4.0),
            "max_anchors": kwargs.get("max_anchors", 3072),
            "confidence_head_alpha": kwargs.get("confidence_head_alpha", 1.0),
            "per_position_loss_weight": kwargs.get("per_position_loss_weight", "fixed-exp-decay"),
            "dpace_alpha": kwargs.get("dpace_alpha", 0.5),
        }
        return dict(shared), dict(shared)

    def forward(self, hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids=None,
                loss_config: LossConfig | None = None, tv_loss_fn=tv_loss, gamma: float = 4.0, max_anchors: int = 3072,
                confidence_head_alpha: float = 1.0, per_position_loss_weight: str = "fixed-exp-decay", dpace_alpha: float = 0.5, **kwargs):
        hidden, logits, targets, aligned, block_index = self._backbone_forward(
            hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids, max_anchors=max_anchors
        )
        blocks, B = max_anchors, self.block_size
        T = input_ids.shape[1]
        block_tokens = input_ids.reshape(-1)[block_index % T].view(blocks, B)
        prev_ids = block_tokens if self.config.sample_from_anchor else torch.cat([block_tokens[:, :1], block_tokens[:, :-1]], dim=1)
        hidden_blocks = hidden.view(blocks, B, -1)
        prev_emb = None
        if self.markov_head is not None:
            prev_emb = self.markov_head.prev_embeddings(prev_ids)
            bias = self.markov_head.block_bias(prev_token_ids=prev_ids, hidden_states=hidden_blocks, prev_emb=prev_emb)
            logits = (logits.view(blocks, B, -1) + bias.to(logits.dtype)).view(1, blocks * B, -1)
        confidence = None
        if self.confidence_head is not None:
            feats = hidden_blocks
            if self.config.confidence_head_with_markov and prev_emb is not None:
                feats = torch.cat([hidden_blocks, prev_emb.to(hidden_blocks.dtype)], dim=-1)
            confidence = self.confidence_head(feats).reshape(1, blocks * B)
        loss, metrics = compute_metrics(
            logits, targets, confidence, aligned, B, loss_config=loss_config or {"kl_div": (kl_div_loss, 1.0)},
            tv_loss_fn=tv_loss_fn, gamma=gamma, confidence_head_alpha=confidence_head_alpha,
            per_position_loss_weight=per_position_loss_weight, dpace_alpha=dpace_alpha,
            sample_from_anchor=self.config.sample_from_anchor,
        )
        return None, loss, metrics
