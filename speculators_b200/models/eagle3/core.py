"""EAGLE-3 draft model with training-time-test (TTT).

Forward semantics follow src/speculators/models/eagle3/core.py:192-365:

1. optional ``input_norm`` (one RMSNorm over the concatenated aux states) or
   per-chunk ``fc_norm``; ``fc: A*H -> H``;
2. targets = ``verifier_lm_head(verifier_norm(verifier_last_hidden_states))``
   without gradient, already in the draft vocabulary;
3. ``ttt_steps`` passes of the decoder stack over the same ``T`` positions.  Pass
   ``s`` feeds ``cat([embed(tokens_s), hidden_{s-1}])`` to the first layer, attends
   to pass 0 causally and to passes ``1..s`` on the diagonal, produces logits,
   a loss against targets shifted by ``s`` (weight ``decay**s``), then teacher
   forcing shifts the ground-truth ids left by ``1 + s`` for the next pass and
   ``position_ids`` advance by one.

What differs from the reference is the execution: the block mask object, the
``DynamicCache`` and ``torch.compile`` are replaced by an ``AttnSpec`` built once
per forward from ``document_ids`` (no host sync), explicit per-pass K/V lists, and
the package's own kernels.  Tensors keep the reference's ``[1, T, ...]`` layout
at the interface and are handled as ``[T, ...]`` inside.
"""

from __future__ import annotations

from typing import ClassVar

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.config import SpeculatorsConfig, VerifierConfig
from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.losses import LossConfig, resolve_loss_config
from speculators_b200.model import DraftVocabMixin, SpeculatorModel
from speculators_b200.models.eagle3.attention import causal_document_interval, ttt_attn_spec
from speculators_b200.models.eagle3.config import Eagle3SpeculatorConfig
from speculators_b200.models.eagle3.metrics import compute_metrics, compute_metrics_from_hidden
from speculators_b200.models.layers import MLP, Attention, DecoderLayer, Linear, RMSNorm, RotaryTable
from speculators_b200.models.utils import resolve_target_layer_ids
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

__all__ = ["Eagle3DraftModel", "Eagle3FirstLayer"]


class Eagle3FirstLayer(nn.Module):
    """Decoder block whose attention reads ``cat([embeds, hidden])`` (2H): both
    halves are normalised separately, the residual is the hidden half (normalised
    when ``norm_before_residual``).  Parity:
    src/speculators/models/eagle3/model_definitions.py:29-110."""

    def __init__(self, config: TransformerLayerConfig, layer_idx: int = 0, norm_before_residual: bool = False):
        super().__init__()
        H = config.hidden_size
        self.hidden_size = H
        self.norm_before_residual = norm_before_residual
        self.self_attn = Attention(config, layer_idx, input_size=2 * H)
        self.mlp = MLP(config)
        self.input_layernorm = RMSNorm(H, config.rms_norm_eps)
        self.hidden_norm = RMSNorm(H, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(H, config.rms_norm_eps)

    def forward(self, embeds, hidden, positions, rotary, spec, past=None, ctx_len=None):
        H = self.hidden_size
        x, normed_hidden = ops.eagle3_input_concat(
            embeds, hidden, self.input_layernorm.weight, self.hidden_norm.weight, self.hidden_norm.variance_epsilon,
            return_hidden_half=True,
        )
        residual = normed_hidden if self.norm_before_residual else hidden
        h = self.self_attn(x, positions, rotary, spec, past, ctx_len, residual=residual)
        return self.mlp(self.post_attention_layernorm(h), residual=h)


@SpeculatorModel.register("eagle3")
class Eagle3DraftModel(DraftVocabMixin, SpeculatorModel):
    config_class: ClassVar[type[Eagle3SpeculatorConfig]] = Eagle3SpeculatorConfig
    _keys_to_ignore_on_load_missing: ClassVar[list[str]] = [
        "embed_tokens.weight", "verifier_norm.weight", "verifier_lm_head.weight", "d2t", "t2d", "input_norm.weight",
    ]
    _keys_to_ignore_on_save: ClassVar[list[str]] = ["verifier_lm_head.weight", "verifier_norm.weight"]
    # forward has fixed shapes and no host synchronisation: a step can be captured in a CUDA graph
    cuda_graph_safe: ClassVar[bool] = True

    def __init__(self, config: Eagle3SpeculatorConfig):
        SpeculatorModel.__init__(self, config)
        self._init_vocab(config)
        tl = config.transformer_layer_config
        H = self.hidden_size
        eps = tl.rms_norm_eps
        self.embed_tokens.weight.requires_grad_(bool(config.embed_requires_grad))

        num_aux = len(config.eagle_aux_hidden_state_layer_ids) if config.eagle_aux_hidden_state_layer_ids else 3
        self.num_aux = num_aux
        self.fc = Linear(num_aux * H, H, bias=False)

        layers: list[nn.Module] = [Eagle3FirstLayer(tl, 0, norm_before_residual=config.norm_before_residual)]
        layers += [DecoderLayer(tl, i) for i in range(1, int(tl.num_hidden_layers))]
        self.layers = nn.ModuleList(layers)

        self.sliding_window = tl.sliding_window
        types = tl.layer_types or []
        self.sliding_window_indices = [i for i, t in enumerate(types) if t == "sliding_attention"]
        self.uses_sliding_window_attn = bool(self.sliding_window_indices)
        self.uses_full_attn = bool(len(layers) - len(self.sliding_window_indices))

        self.rotary_emb = RotaryTable(tl)
        self.norm = RMSNorm(H, eps)
        self.verifier_norm = RMSNorm(H, eps)
        self.verifier_norm.weight.requires_grad_(False)
        self.input_norm = RMSNorm(num_aux * H, eps) if config.norm_before_fc else None
        self.fc_norm = nn.ModuleList([RMSNorm(H, eps) for _ in range(num_aux)]) if config.fc_norm else None

    @property
    def target_layer_ids(self) -> list[int]:
        return self.config.eagle_aux_hidden_state_layer_ids

    # ------------------------------------------------------------------ loading
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, *args, **kwargs):
        model = super().from_pretrained(pretrained_model_name_or_path, *args, **kwargs)
        verifier_path = model.config.speculators_config.verifier.name_or_path if model.config.speculators_config else None
        if verifier_path is not None and model.config.eagle_aux_hidden_state_layer_ids is None:
            model.config.eagle_aux_hidden_state_layer_ids = resolve_target_layer_ids(None, verifier_path)
        return model

    def load_verifier_weights(self):
        super().load_verifier_weights()
        self.embed_tokens.weight.requires_grad_(bool(self.config.embed_requires_grad))
        spec_cfg = self.config.speculators_config
        if spec_cfg is None or spec_cfg.verifier.name_or_path is None:
            return
        from speculators_b200.models.utils import get_verifier_config

        vh = get_verifier_config(spec_cfg.verifier.name_or_path).hidden_size
        if vh != self.hidden_size:
            raise ValueError(f"Verifier hidden size {vh} does not match draft hidden size {self.hidden_size}.")

    # ------------------------------------------------------------------ forward
    def _project_aux(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if self.input_norm is not None:
            hidden_states = self.input_norm(hidden_states)
        if self.fc_norm is not None:
            chunks = hidden_states.chunk(len(self.fc_norm), dim=-1)
            hidden_states = torch.cat([n(c) for n, c in zip(self.fc_norm, chunks, strict=True)], dim=-1)
        return self.fc(hidden_states)

    def forward(
        self,
        hidden_states: torch.Tensor,  # [1, T, A*H]
        input_ids: torch.Tensor,  # [1, T]
        document_ids: torch.Tensor,  # [1, T]
        loss_mask: torch.Tensor | None = None,  # [1, T]
        position_ids: torch.Tensor | None = None,  # [1, T]
        verifier_last_hidden_states: torch.Tensor | None = None,  # [1, T, H]
        ttt_steps: int = 3,
        ttt_step_loss_decay: float = 1.0,
        loss_config: LossConfig | None = None,
        return_draft_tokens: bool = True,
        **_,
    ):
        """``return_draft_tokens=False`` (what the trainer passes) skips the per-pass
        argmax over the full ``[T, V]`` logits; the first element of the result is
        then an empty list."""
        device = hidden_states.device
        T = hidden_states.shape[1]
        dtype = self.fc.weight.dtype
        positions = (
            position_ids.reshape(-1).to(torch.long) if position_ids is not None
            else torch.arange(1, T + 1, dtype=torch.long, device=device)
        )
        doc = document_ids.reshape(-1).to(device)
        ids = input_ids.reshape(-1)
        original_ids = ids

        full_iv = causal_document_interval(doc, None) if self.uses_full_attn else None
        win_iv = causal_document_interval(doc, self.sliding_window) if self.uses_sliding_window_attn else None

        hidden = self._project_aux(hidden_states.reshape(T, -1).to(dtype))

        return_loss = verifier_last_hidden_states is not None
        if return_loss:
            with torch.no_grad():
                vl = verifier_last_hidden_states.reshape(T, -1).to(dtype)
                targets = ops.linear(self.verifier_norm(vl), self.verifier_lm_head.weight)  # [T, Vd]
            loss = torch.zeros((), device=device, dtype=torch.float32)
            prev_correct = (
                loss_mask.to(torch.bool).clone() if loss_mask is not None
                else torch.ones(1, T, device=device, dtype=torch.bool)
            )
            metrics: dict[str, torch.Tensor] = {}

        past = [[] for _ in self.layers]
        draft_tokens = []
        # teacher forcing: pass k reads the ground-truth ids shifted left by k (zero padded);
        # one padded copy, every pass takes a view of it
        padded_ids = torch.cat([original_ids, original_ids.new_zeros(ttt_steps)])
        for step in range(ttt_steps):
            with torch.no_grad():
                embeds = self.embed_tokens(ids).to(dtype)
            full_spec = ttt_attn_spec(doc, step, interval=full_iv) if full_iv is not None else None
            win_spec = ttt_attn_spec(doc, step, interval=win_iv) if win_iv is not None else None
            for li, layer in enumerate(self.layers):
                spec = win_spec if li in self.sliding_window_indices else full_spec
                if li == 0:
                    hidden = layer(embeds, hidden, positions, self.rotary_emb, spec, past[li])
                else:
                    hidden = layer(hidden, positions, self.rotary_emb, spec, past[li])
            if self.config.norm_output:
                hidden = head_in = self.norm(hidden)
            else:
                head_in = self.norm(hidden)
            fused = None
            if return_loss and not return_draft_tokens:
                # lm_head GEMM with the loss's forward reduction in its epilogue (CUDA, bf16, KL / CE)
                fused = compute_metrics_from_hidden(
                    head_in, self.lm_head.weight, targets.unsqueeze(0), loss_mask, prev_correct, step, ttt_step_loss_decay,
                    loss_config=loss_config,
                )
            if fused is None:
                logits = ops.linear(head_in, self.lm_head.weight)
                if return_loss:
                    fused = compute_metrics(
                        logits.unsqueeze(0), targets.unsqueeze(0), loss_mask, prev_correct, step,
                        ttt_step_loss_decay, loss_config=loss_config,
                    )
            if return_loss:
                loss = loss + fused[0]
                metrics.update(fused[1])

            if return_draft_tokens:
                draft_tokens.append(torch.argmax(logits.detach(), dim=-1).unsqueeze(0))
            ids = padded_ids[1 + step : 1 + step + T]
            positions = positions + 1

        if return_loss:
            metrics["loss_sum"] = loss.detach().clone()
            metrics["loss_total"] = torch.ones((), device=device)
            return draft_tokens, loss, metrics
        return draft_tokens

    # ------------------------------------------------------------------ training glue
    @classmethod
    def from_training_args(cls, verifier_config, t2d: torch.Tensor | None = None, d2t: torch.Tensor | None = None, **kwargs) -> "Eagle3DraftModel":
        target_layer_ids = resolve_target_layer_ids(
            kwargs.get("target_layer_ids"), kwargs["verifier_name_or_path"], trust_remote_code=kwargs.get("trust_remote_code", False)
        )
        config = Eagle3SpeculatorConfig(
            transformer_layer_config=verifier_config,
            draft_vocab_size=kwargs["draft_vocab_size"],
            norm_before_residual=kwargs["norm_before_residual"],
            norm_before_fc=kwargs.get("norm_before_fc", False),
            fc_norm=kwargs.get("fc_norm", False),
            norm_output=kwargs.get("norm_output", False),
            embed_requires_grad=kwargs.get("embed_requires_grad", False),
            eagle_aux_hidden_state_layer_ids=target_layer_ids,
            speculators_config=SpeculatorsConfig(
                algorithm="eagle3",
                proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=kwargs["ttt_steps"])],
                default_proposal_method="greedy",
                verifier=VerifierConfig.from_pretrained(kwargs["verifier_name_or_path"]),
            ),
        )
        model = cls(config=config)
        model.load_vocab_mappings(t2d, d2t)
        model.load_verifier_weights()
        return model

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        loss_config = resolve_loss_config(kwargs["loss_fn"], kwargs.get("loss_implementation", "fused"))
        call = {
            "ttt_steps": kwargs["ttt_steps"],
            "ttt_step_loss_decay": kwargs["ttt_step_loss_decay"],
            "loss_config": loss_config,
            "return_draft_tokens": False,  # the trainer only consumes loss and metrics
        }
        return dict(call), dict(call)
