"""P-EAGLE draft: EAGLE-3 architecture trained with parallel multi-depth
prediction instead of the sequential TTT loop.

One forward pass over the COD samples (``peagle/data.py``): depth-0 rows carry the
real token and real aux hidden states, deeper rows carry ``mask_token_id`` and the
learnable ``mask_hidden`` vector; a single pass through the decoder stack with the
rollout mask (``peagle/attention.py``); targets are the verifier logits gathered
at ``anchor + depth``.  Semantics: src/speculators/models/peagle/core.py:53-206.
"""

from __future__ import annotations

from typing import ClassVar

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.config import SpeculatorsConfig, VerifierConfig
from speculators_b200.losses import LossConfig, resolve_loss_config
from speculators_b200.model import SpeculatorModel
from speculators_b200.models.eagle3.core import Eagle3DraftModel
from speculators_b200.models.peagle.attention import peagle_attn_spec
from speculators_b200.models.peagle.config import PEagleSpeculatorConfig
from speculators_b200.models.peagle.data import generate_cod_sample_indices, generate_cod_sample_indices_fixed
from speculators_b200.models.peagle.metrics import compute_metrics
from speculators_b200.models.utils import resolve_target_layer_ids
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

__all__ = ["PEagleDraftModel"]


def _fixed_shape_default(explicit: bool | None) -> bool:
    """COD sampling with argument-only shapes: the explicit choice, else ``SB200_PEAGLE_FIXED_SHAPE=1``.

    Opt-in because the fixed shapes are sized for a full loss mask: on the 70B-shaped benchmark row
    (about half of the positions inside the mask) the padded sampler's step, replayed as a CUDA graph, took
    53.9 ms against 44.1 ms for the variable-shape sampler's eager step on the same GPU - the padding rows cost
    more than the launch gaps save.  It pays when most positions are supervised."""
    import os

    return bool(explicit) if explicit is not None else os.environ.get("SB200_PEAGLE_FIXED_SHAPE") == "1"


@SpeculatorModel.register("peagle")
class PEagleDraftModel(Eagle3DraftModel):
    config_class: ClassVar[type[PEagleSpeculatorConfig]] = PEagleSpeculatorConfig
    _keys_to_ignore_on_load_missing: ClassVar[list[str]] = [*Eagle3DraftModel._keys_to_ignore_on_load_missing, "mask_hidden"]
    # the variable-shape COD sampler produces data-dependent row counts
    cuda_graph_safe: ClassVar[bool] = False

    def __init__(self, config: PEagleSpeculatorConfig):
        super().__init__(config)
        # with the fixed-shape sampler every tensor shape of the step is static (decided per call: ``graph_safe_with``)
        self.cuda_graph_safe = True
        self.mask_token_id = config.mask_token_id
        self.mask_hidden = nn.Parameter(torch.randn(1, 1, self.num_aux * self.hidden_size))

    def forward(
        self, hidden_states, input_ids, document_ids, position_ids=None, loss_mask=None, verifier_last_hidden_states=None,
        loss_config: LossConfig | None = None, max_anchors: int | None = None, num_depths: int = 8,
        down_sample_ratio: float = 0.7, down_sample_ratio_min: float = 0.2, fixed_shape: bool = False, cod_sample=None, **_,
    ):
        """``fixed_shape``: draw the COD sample with shapes that depend only on the
        arguments (rows the mask rules out are carried as inert padding), which makes the
        step capturable in a CUDA graph.  ``cod_sample``: a ready
        ``(anchor_pos, depth[, row_valid])`` to use instead of drawing one."""
        if verifier_last_hidden_states is None:
            raise ValueError("verifier_last_hidden_states required for training")
        if self.mask_token_id is None:
            raise ValueError("mask_token_id is not set on the config; pass --mask-token-id")
        device = hidden_states.device
        T = input_ids.shape[1]
        dtype = self.fc.weight.dtype
        if loss_mask is None:
            loss_mask = torch.ones_like(input_ids, dtype=torch.float32)
        row_valid = None
        if cod_sample is not None:
            anchor_pos, depth, *rest = cod_sample
            row_valid = rest[0] if rest else None
        elif fixed_shape:
            anchor_pos, depth, row_valid = generate_cod_sample_indices_fixed(
                T, loss_mask, num_depths=num_depths, down_sample_ratio=down_sample_ratio,
                down_sample_ratio_min=down_sample_ratio_min, max_anchors=max_anchors,
            )
        else:
            anchor_pos, depth = generate_cod_sample_indices(
                T, loss_mask, num_depths=num_depths, down_sample_ratio=down_sample_ratio,
                down_sample_ratio_min=down_sample_ratio_min, max_anchors=max_anchors,
            )
        orig = anchor_pos + depth
        depth0 = depth == 0
        ids = torch.where(depth0, input_ids.reshape(-1)[orig], torch.full_like(orig, self.mask_token_id))
        embeds = self.embed_tokens(ids).to(dtype)
        aux = hidden_states.reshape(T, -1).to(dtype)
        sampled = torch.where(depth0.unsqueeze(-1), aux[orig], self.mask_hidden.reshape(1, -1).to(dtype).expand(orig.shape[0], -1))
        hidden = self._project_aux(sampled)

        doc = document_ids.reshape(-1).to(device)
        full_spec = peagle_attn_spec(anchor_pos, depth, doc, num_depths, None, row_valid) if self.uses_full_attn else None
        win_spec = (peagle_attn_spec(anchor_pos, depth, doc, num_depths, self.sliding_window, row_valid)
                    if self.uses_sliding_window_attn else None)
        self.rotary_emb.ensure(int(T) + num_depths + 1)
        for li, layer in enumerate(self.layers):
            spec = win_spec if li in self.sliding_window_indices else full_spec
            if li == 0:
                hidden = layer(embeds, hidden, orig, self.rotary_emb, spec, None, T)
            else:
                hidden = layer(hidden, orig, self.rotary_emb, spec, None, T)
        logits = ops.linear(self.norm(hidden), self.lm_head.weight)
        with torch.no_grad():
            vl = verifier_last_hidden_states.reshape(T, -1).to(dtype)[orig]
            targets = ops.linear(self.verifier_norm(vl), self.verifier_lm_head.weight)
        loss, metrics = compute_metrics(
            logits.unsqueeze(0), targets.unsqueeze(0), loss_mask, anchor_pos, depth, num_depths, loss_config=loss_config,
            row_valid=row_valid,
        )
        return None, loss, metrics

    @classmethod
    def from_training_args(cls, verifier_config, t2d=None, d2t=None, **kwargs) -> "PEagleDraftModel":
        target_layer_ids = resolve_target_layer_ids(
            kwargs.get("target_layer_ids"), kwargs["verifier_name_or_path"], trust_remote_code=kwargs.get("trust_remote_code", False)
        )
        config = PEagleSpeculatorConfig(
            transformer_layer_config=verifier_config,
            draft_vocab_size=kwargs["draft_vocab_size"],
            norm_before_residual=kwargs.get("norm_before_residual", False),
            norm_before_fc=kwargs.get("norm_before_fc", False),
            fc_norm=kwargs.get("fc_norm", False),
            norm_output=kwargs.get("norm_output", False),
            eagle_aux_hidden_state_layer_ids=target_layer_ids,
            mask_token_id=kwargs.get("mask_token_id"),
            speculators_config=SpeculatorsConfig(
                algorithm="peagle",
                proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=kwargs.get("num_depths", 8))],
                default_proposal_method="greedy",
                verifier=VerifierConfig.from_pretrained(kwargs["verifier_name_or_path"]),
            ),
        )
        model = cls(config=config)
        model.load_vocab_mappings(t2d, d2t)
        model.load_verifier_weights()
        return model

    def graph_safe_with(self, call_kwargs: dict) -> bool:
        """Whether a step called with ``call_kwargs`` has static shapes: only with the fixed-shape sampler."""
        return bool(call_kwargs.get("fixed_shape"))

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        shared = {
            "loss_config": resolve_loss_config(kwargs["loss_fn"], kwargs.get("loss_implementation", "fused")),
            "max_anchors": kwargs.get("max_anchors"),
            "num_depths": kwargs.get("num_depths", 8),
            "down_sample_ratio": kwargs.get("down_sample_ratio", 0.7),
            "down_sample_ratio_min": kwargs.get("down_sample_ratio_min", 0.2),
            "fixed_shape": _fixed_shape_default(kwargs.get("cod_fixed_shape")),
        }
        return dict(shared), dict(shared)
