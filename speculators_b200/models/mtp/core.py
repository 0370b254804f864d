"""MTP draft model: fine-tunes a verifier's native multi-token-prediction head.

Teacher-forced recursion over ``K`` steps (src/speculators/models/mtp/core.py:
114-231): with ``valid_len = T - K - 1``, step ``k`` combines the hidden states of
the previous step (the verifier's last hidden states at step 0) with the
embeddings of ``input_ids[k+1 : k+1+valid_len]``, runs the MTP layer under a plain
causal mask, and is trained with cross-entropy against ``input_ids[k+2 : ...]``
(positions outside ``loss_mask`` ignored) weighted ``beta**k / sum_j beta**j``.
The full verifier vocabulary is used; ``embed_tokens`` / ``lm_head`` come from the
verifier and are not saved.
"""

from __future__ import annotations

from typing import Any, ClassVar

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.config import SpeculatorsConfig, VerifierConfig
from speculators_b200.model import DraftVocabMixin, SpeculatorModel
from speculators_b200.models.layers import RotaryTable
from speculators_b200.models.mtp.config import MTPSpeculatorConfig
from speculators_b200.models.mtp.model_definitions import build_mtp_layer
from speculators_b200.ops import AttnSpec
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

__all__ = ["MTPDraftModel", "compute_step_weights"]


def _expert_parallel_group(expert_parallel: bool | None):
    import os

    import torch.distributed as dist

    if expert_parallel is None:
        expert_parallel = os.environ.get("SB200_EXPERT_PARALLEL", "0") == "1"
    if not expert_parallel or not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return None
    return dist.group.WORLD


def compute_step_weights(beta: float = 0.6, num_steps: int = 3) -> list[float]:
    """``beta**k`` normalised to sum to one (FastMTP, arXiv:2509.18362, eq. 2)."""
    raw = [beta**k for k in range(num_steps)]
    total = sum(raw)
    return [w / total for w in raw]


@SpeculatorModel.register("mtp")
class MTPDraftModel(DraftVocabMixin, SpeculatorModel):
    config_class: ClassVar[type[MTPSpeculatorConfig]] = MTPSpeculatorConfig
    _keys_to_ignore_on_save: ClassVar[list[str]] = ["embed_tokens.weight", "lm_head.weight", "verifier_lm_head.weight"]
    _keys_to_ignore_on_load_missing: ClassVar[list[str]] = ["embed_tokens.weight", "lm_head.weight", "verifier_lm_head.weight", "t2d", "d2t"]
    cuda_graph_safe: ClassVar[bool] = True

    def __init__(self, config: MTPSpeculatorConfig, ep_group=None):
        """``ep_group`` (mixture-of-experts heads only): split the experts over this process group
        instead of keeping all of them on every rank; tokens then travel to their experts' ranks
        and back inside the layer (``models/moe.py``), and the training engine treats the expert
        tensors as rank-local.  The reference only replicates or FSDP-shards the experts."""
        SpeculatorModel.__init__(self, config)
        self._init_vocab(config)
        if self.use_draft_vocab:
            raise NotImplementedError("Vocab reduction is not supported for MTP speculators")
        tc = config.transformer_layer_config
        self.mtp_layers = nn.ModuleList([build_mtp_layer(tc, 0, ep_group=ep_group)])
        # a dense layer has fixed shapes; so has a layer with experts that all live on this rank (the grouped
        # GEMMs take the routing counts from device memory).  The expert-parallel exchange sizes its plan from
        # counts read on the host, so those steps run eagerly.
        self.cuda_graph_safe = type(self.mtp_layers[0]).__name__ != "MoEMTPLayer" or ep_group is None
        self.rotary_emb = RotaryTable(tc)

    @property
    def layers(self) -> nn.ModuleList:
        return self.mtp_layers

    @property
    def target_layer_ids(self) -> list[int]:
        return [int(self.config.transformer_layer_config.num_hidden_layers)]

    def load_verifier_weights(self) -> None:
        with torch.no_grad():
            self.embed_tokens.weight.fill_(float("nan"))
            self.lm_head.weight.fill_(float("nan"))
        super().load_verifier_weights()
        if hasattr(self, "verifier_lm_head"):
            del self.verifier_lm_head  # MTP trains against token ids, not verifier logits

    def forward(self, input_ids, hidden_states, attention_mask=None, position_ids=None, loss_mask=None,
                step_weights: list[float] | None = None, return_dict: bool = True, **_: Any):
        del attention_mask, return_dict
        ids = input_ids.reshape(-1).long()
        device = ids.device
        T = ids.shape[0]
        dtype = self.lm_head.weight.dtype
        num_steps = self.config.num_speculative_steps
        if step_weights is not None and len(step_weights) != num_steps:
            raise ValueError(
                f"step_weights has {len(step_weights)} entries but num_speculative_steps={num_steps}; "
                f"expected exactly {num_steps} weights."
            )
        positions = position_ids.reshape(-1).long() if position_ids is not None else torch.arange(T, device=device)
        all_logits: list[torch.Tensor] = []
        total = torch.zeros((), device=device, dtype=torch.float32)
        metrics: dict[str, torch.Tensor] = {}
        steps = min(num_steps, max(0, T - 2))
        valid_len = T - steps - 1
        if valid_len <= 0 or steps == 0:
            metrics["loss_sum"] = total.detach().clone()
            metrics["loss_total"] = torch.ones((), device=device)
            return all_logits, total, metrics
        pos = positions[:valid_len]
        idx = torch.arange(valid_len, device=device, dtype=torch.int32)
        spec = AttnSpec(lo=torch.zeros_like(idx), hi=idx + 1)  # plain causal, as in the reference
        current = hidden_states.reshape(T, -1).to(dtype)
        mask = loss_mask.reshape(-1) if loss_mask is not None else None
        for step in range(steps):
            with torch.no_grad():
                emb = self.embed_tokens(ids[step + 1 : step + 1 + valid_len]).to(dtype)
            out = self.mtp_layers[0](current[:valid_len], emb, pos, self.rotary_emb, spec)
            logits = ops.linear(out, self.lm_head.weight)
            all_logits.append(logits.unsqueeze(0))
            labels = ids[step + 2 : step + 2 + valid_len]
            keep = mask[step + 2 : step + 2 + valid_len] != 0 if mask is not None else torch.ones_like(labels, dtype=torch.bool)
            per_row = ops.token_cross_entropy(logits, labels, keep)
            weight = step_weights[step] if step_weights is not None else 1.0
            step_loss = weight * per_row.sum() / keep.sum().clamp(min=1)
            total = total + step_loss
            metrics[f"loss_step_{step}"] = step_loss.detach().clone()
            current = out
        metrics["loss_sum"] = total.detach().clone()
        metrics["loss_total"] = torch.ones((), device=device)
        return all_logits, total, metrics

    @classmethod
    def from_training_args(cls, verifier_config, *, num_speculative_steps: int = 3, verifier_name_or_path: str | None = None,
                           expert_parallel: bool | None = None, **_: Any) -> "MTPDraftModel":
        """``expert_parallel`` (default: the environment variable ``SB200_EXPERT_PARALLEL=1``): split a
        mixture-of-experts head's experts over all ranks of the job."""
        if verifier_name_or_path is None:
            raise ValueError(
                "verifier_name_or_path is required for MTP training. The verifier model must contain native MTP "
                "weights (mtp.* keys) to extract."
            )
        config = MTPSpeculatorConfig(
            transformer_layer_config=verifier_config,
            speculators_config=SpeculatorsConfig(
                algorithm="mtp",
                proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=num_speculative_steps)],
                default_proposal_method="greedy",
                verifier=VerifierConfig.from_pretrained(verifier_name_or_path),
            ),
        )
        model = cls(config=config, ep_group=_expert_parallel_group(expert_parallel))
        from speculators_b200.convert.mtp.converter import MTPConverter

        state = MTPConverter().convert_to_state_dict(verifier_name_or_path)
        model.load_state_dict(state, strict=False)
        model.load_verifier_weights()
        return model

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        weights = kwargs.get("step_weights")
        if weights is None:
            if "num_speculative_steps" not in kwargs:
                raise ValueError("num_speculative_steps must be set from the model config before calling get_trainer_kwargs")
            weights = compute_step_weights(beta=kwargs.get("step_weight_beta", 0.6), num_steps=kwargs["num_speculative_steps"])
        call: dict[str, Any] = {"step_weights": weights}
        return call, dict(call)
