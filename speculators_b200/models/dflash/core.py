"""DFlash draft model: anchored-block parallel drafting.

``max_anchors`` anchor positions are drawn from the loss mask; each anchor spawns
a block of ``block_size`` query tokens (slot 0 = the anchor's own token, the rest
``mask_token_id``).  The blocks run through ``num_hidden_layers`` DFlash decoder
blocks whose keys/values are the projected verifier states ``hidden_norm(fc(aux))``
plus the block itself; the logits of slot ``k`` are trained against the verifier
logits at ``anchor + k`` (``sample_from_anchor``) or ``anchor + k - 1``.  Semantics:
src/speculators/models/dflash/core.py:330-478.  All shapes are fixed by
``max_anchors`` and ``block_size`` and nothing is read back to the host.
"""

from __future__ import annotations

import logging
from typing import ClassVar

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.config import SpeculatorsConfig, VerifierConfig
from speculators_b200.losses import LossConfig, resolve_loss_config
from speculators_b200.model import DraftVocabMixin, SpeculatorModel
from speculators_b200.models.dflash.attention import anchor_block_attn_spec
from speculators_b200.models.dflash.config import DFlashSpeculatorConfig
from speculators_b200.models.dflash.metrics import compute_metrics
from speculators_b200.models.dflash.model_definitions import DFlashDecoderLayer
from speculators_b200.models.dflash.utils import get_base_indices_for_anchored_blocks, select_anchors
from speculators_b200.models.layers import Linear, RMSNorm, RotaryTable
from speculators_b200.models.utils import resolve_target_layer_ids
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

log = logging.getLogger("speculators")

__all__ = ["DFlashDraftModel"]


@SpeculatorModel.register("dflash")
class DFlashDraftModel(DraftVocabMixin, SpeculatorModel):
    config_class: ClassVar[type[DFlashSpeculatorConfig]] = DFlashSpeculatorConfig
    _keys_to_ignore_on_load_missing: ClassVar[list[str]] = ["embed_tokens.weight", "verifier_norm.weight", "verifier_lm_head.weight", "t2d", "d2t"]
    _keys_to_ignore_on_save: ClassVar[list[str]] = ["verifier_lm_head.weight", "verifier_norm.weight"]
    cuda_graph_safe: ClassVar[bool] = True

    def __init__(self, config: DFlashSpeculatorConfig):
        SpeculatorModel.__init__(self, config)
        self._init_vocab(config)
        tl = config.transformer_layer_config
        H, eps = tl.hidden_size, tl.rms_norm_eps
        n_layers = int(tl.num_hidden_layers)
        self.layers = nn.ModuleList([DFlashDecoderLayer(tl, i) for i in range(n_layers)])
        self.sliding_window = tl.sliding_window
        self.sliding_window_indices = [i for i, t in enumerate(tl.layer_types or []) if t == "sliding_attention"]
        self.uses_sliding_window_attn = bool(self.sliding_window_indices)
        self.uses_full_attn = bool(n_layers - len(self.sliding_window_indices))
        self.sliding_window_non_causal = config.sliding_window_non_causal
        self.norm = RMSNorm(H, eps)
        self.rotary_emb = RotaryTable(tl)
        self.fc = Linear(len(self.target_layer_ids or [0, 0, 0]) * H, H, bias=False)
        self.hidden_norm = RMSNorm(H, eps)
        self.verifier_norm = RMSNorm(H, eps)
        self.verifier_norm.weight.requires_grad_(False)
        self.block_size = config.block_size
        if type(self).__name__ == "DFlashDraftModel" and config.sample_from_anchor:
            log.warning(
                "DFlash with sample_from_anchor=True may not be supported in all inference engines (e.g., vLLM). "
                "Verify compatibility with your deployment target."
            )

    @property
    def target_layer_ids(self) -> list[int]:
        return self.config.aux_hidden_state_layer_ids

    @property
    def mask_token_id(self) -> int:
        if self.config.mask_token_id is None:
            raise ValueError(
                "mask_token_id is not set on the config. Pass --mask-token-id during training or ensure the "
                "config was saved with mask_token_id set."
            )
        return self.config.mask_token_id

    # ------------------------------------------------------------------ backbone
    def _backbone_forward(self, hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids=None, **kwargs):
        """-> ``(hidden, logits, targets, aligned_loss_mask, anchored_block_indices)``;
        ``hidden`` / ``logits`` / ``targets`` are ``[1, N*B, .]``."""
        device = hidden_states.device
        T = hidden_states.shape[1]
        dtype = self.fc.weight.dtype
        B = self.block_size
        num_anchors = kwargs.pop("max_anchors", 512)
        positions = position_ids.reshape(-1).long() if position_ids is not None else torch.arange(T, dtype=torch.long, device=device)
        doc = document_ids.reshape(-1).to(device)
        ids = input_ids.reshape(-1)

        anchors, anchor_valid = select_anchors(loss_mask, num_anchors, B)
        full_spec = anchor_block_attn_spec(doc, anchors, B, None) if self.uses_full_attn else None
        win_spec = (
            anchor_block_attn_spec(doc, anchors, B, self.sliding_window, self.sliding_window_non_causal)
            if self.uses_sliding_window_attn else None
        )
        block_ids = torch.full((num_anchors * B,), self.mask_token_id, dtype=torch.long, device=device)
        block_ids[::B] = ids[anchors]
        noise = self.embed_tokens(block_ids).to(dtype)
        context = self.hidden_norm(self.fc(hidden_states.reshape(T, -1).to(dtype)))
        noise_positions = get_base_indices_for_anchored_blocks(positions[anchors], B)
        all_positions = torch.cat([positions, noise_positions])
        block_index = get_base_indices_for_anchored_blocks(anchors, B)
        target_index = (block_index if self.config.sample_from_anchor else block_index - 1) % T
        with torch.no_grad():
            vl = verifier_last_hidden_states.reshape(T, -1).to(dtype)[target_index]
            targets = ops.linear(self.verifier_norm(vl), self.verifier_lm_head.weight)
        for li, layer in enumerate(self.layers):
            spec = win_spec if li in self.sliding_window_indices else full_spec
            noise = layer(noise, context, noise_positions, all_positions, self.rotary_emb, spec)
        hidden = self.norm(noise)
        logits = ops.linear(hidden, self.lm_head.weight)
        aligned = loss_mask.reshape(-1)[block_index % T].clone()
        aligned = aligned * anchor_valid.repeat_interleave(B).to(aligned.dtype)
        aligned = aligned * (block_index < T).to(aligned.dtype)
        if not self.config.sample_from_anchor:
            aligned[::B] = 0
        return hidden.unsqueeze(0), logits.unsqueeze(0), targets.unsqueeze(0), aligned.unsqueeze(0), block_index

    def forward(self, hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids=None,
                loss_config: LossConfig | None = None, gamma: float = 4.0, max_anchors: int = 512,
                per_position_loss_weight: str = "fixed-exp-decay", dpace_alpha: float = 0.5, **kwargs):
        _, logits, targets, aligned, _ = self._backbone_forward(
            hidden_states, input_ids, loss_mask, verifier_last_hidden_states, document_ids, position_ids, max_anchors=max_anchors
        )
        loss, metrics = compute_metrics(
            logits, targets, aligned, self.block_size, gamma=gamma, loss_config=loss_config,
            per_position_loss_weight=per_position_loss_weight, dpace_alpha=dpace_alpha,
            sample_from_anchor=self.config.sample_from_anchor,
        )
        return None, loss, metrics

    # ------------------------------------------------------------------ training glue
    @staticmethod
    def _build_base_config_kwargs(algorithm: str, verifier_config, **kwargs) -> dict:
        target_layer_ids = resolve_target_layer_ids(
            kwargs.get("target_layer_ids"), kwargs["verifier_name_or_path"], trust_remote_code=kwargs.get("trust_remote_code", False)
        )
        block_size = kwargs.get("block_size", 8)
        sfa = kwargs.get("sample_from_anchor")
        sample_from_anchor = (algorithm == "dspark") if sfa is None else sfa
        return {
            "transformer_layer_config": verifier_config,
            "draft_vocab_size": kwargs["draft_vocab_size"],
            "block_size": block_size,
            "aux_hidden_state_layer_ids": target_layer_ids,
            "mask_token_id": kwargs.get("mask_token_id"),
            "sliding_window_non_causal": kwargs.get("sliding_window_non_causal", False),
            "sample_from_anchor": sample_from_anchor,
            "speculators_config": SpeculatorsConfig(
                algorithm=algorithm,
                proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=block_size if sample_from_anchor else block_size - 1)],
                default_proposal_method="greedy",
                verifier=VerifierConfig.from_pretrained(kwargs["verifier_name_or_path"]),
            ),
        }

    @classmethod
    def from_training_args(cls, verifier_config, t2d=None, d2t=None, **kwargs) -> "DFlashDraftModel":
        model = cls(config=DFlashSpeculatorConfig(**cls._build_base_config_kwargs("dflash", verifier_config, **kwargs)))
        model.load_vocab_mappings(t2d, d2t)
        model.load_verifier_weights()
        return model

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        shared = {
            "loss_config": resolve_loss_config(kwargs["loss_fn"], kwargs.get("loss_implementation", "fused")),
            "gamma": kwargs.get("dflash_decay_gamma", 4.0),
            "max_anchors": kwargs.get("max_anchors", 512),
            "per_position_loss_weight": kwargs.get("per_position_loss_weight", "fixed-exp-decay"),
            "dpace_alpha": kwargs.get("dpace_alpha", 0.5),
        }
        return dict(shared), dict(shared)
