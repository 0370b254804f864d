"""Research EAGLE-3 checkpoint -> speculators format.

The research layout names the single decoder layer ``midlayer.*``; everything else
already matches.  The converter renames ``midlayer.`` to ``layers.0.``, builds an
``Eagle3SpeculatorConfig`` (Llama decoder description from the source config,
target vocabulary from ``t2d`` when present, else from the verifier) and writes
``config.json`` + ``model.safetensors``.  Parity:
src/speculators/convert/eagle/eagle3_converter.py:44-242.
"""

from __future__ import annotations

import logging
from pathlib import Path

from speculators_b200.config import SpeculatorsConfig, VerifierConfig
from speculators_b200.convert.utils import ensure_checkpoint_is_local, find_vocab_size, load_checkpoint_config, load_checkpoint_weights
from speculators_b200.layer_config import read_config_json
from speculators_b200.models.eagle3 import Eagle3DraftModel, Eagle3SpeculatorConfig
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

log = logging.getLogger("speculators")

__all__ = ["Eagle3Converter"]


class Eagle3Converter:
    def convert(self, input_path, output_path, base_model: str, validate: bool = True, norm_before_residual: bool = False,
                norm_before_fc: bool = False, fc_norm: bool = False, norm_output: bool = False,
                eagle_aux_hidden_state_layer_ids: list[int] | None = None, cache_dir=None) -> None:
        local = ensure_checkpoint_is_local(input_path, cache_dir)
        source = load_checkpoint_config(local)
        weights = load_checkpoint_weights(local)
        log.info("Converting Eagle-3 checkpoint %s (%d tensors)", input_path, len(weights))
        if "t2d" in weights:
            source["target_vocab_size"] = weights["t2d"].shape[0]
        else:
            vocab = find_vocab_size(read_config_json(base_model))
            if vocab is None:
                raise ValueError("Could not determine vocab_size from target model config.")
            source["target_vocab_size"] = vocab
        config = self._build_config(source, base_model, norm_before_residual, norm_before_fc, fc_norm, norm_output, eagle_aux_hidden_state_layer_ids)
        saved = self._save(config, weights, output_path)
        log.info("Saved to: %s", saved)
        if validate:
            Eagle3DraftModel.from_pretrained(str(saved))

    @staticmethod
    def _decoder_config(source: dict, base_model: str) -> dict:
        target = read_config_json(base_model)
        cfg = {
            "model_type": "llama", "vocab_size": source.get("target_vocab_size", 128000), "hidden_size": source.get("hidden_size", 4096),
            "intermediate_size": source.get("intermediate_size", 11008), "num_hidden_layers": source.get("num_hidden_layers", 1),
            "num_attention_heads": source.get("num_attention_heads", 32), "num_key_value_heads": source.get("num_key_value_heads", 8),
            "hidden_act": source.get("hidden_act", "silu"),
            "max_position_embeddings": max(source.get("max_position_embeddings", 4096), target.get("max_position_embeddings", 4096)),
            "initializer_range": source.get("initializer_range", 0.02), "rms_norm_eps": source.get("rms_norm_eps", 1e-6),
            "attention_bias": source.get("attention_bias", False), "mlp_bias": source.get("mlp_bias", False),
            "tie_word_embeddings": False, "rope_theta": source.get("rope_theta", 10000.0),
        }
        if source.get("head_dim"):
            cfg["head_dim"] = source["head_dim"]
        if source.get("rope_scaling"):
            cfg["rope_scaling"] = source["rope_scaling"]
        return cfg

    def _build_config(self, source, base_model, norm_before_residual, norm_before_fc, fc_norm, norm_output, aux_ids) -> Eagle3SpeculatorConfig:
        verifier_cfg = read_config_json(base_model)
        return Eagle3SpeculatorConfig(
            transformer_layer_config=self._decoder_config(source, base_model),
            speculators_config=SpeculatorsConfig(
                algorithm="eagle3", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=3)], default_proposal_method="greedy",
                verifier=VerifierConfig(name_or_path=base_model, architectures=verifier_cfg.get("architectures", ["LlamaForCausalLM"])),
            ),
            draft_vocab_size=source.get("draft_vocab_size", 32000), norm_before_residual=norm_before_residual,
            norm_before_fc=norm_before_fc or source.get("norm_before_fc", False), fc_norm=fc_norm or source.get("fc_norm", False),
            norm_output=norm_output or source.get("norm_output", False), target_hidden_size=source.get("target_hidden_size"),
            eagle_aux_hidden_state_layer_ids=aux_ids,
        )

    @staticmethod
    def remap_keys(weights: dict) -> dict:
        return {(("layers.0." + k[len("midlayer."):]) if k.startswith("midlayer.") else k): v for k, v in weights.items()}

    def _save(self, config, weights, output_dir) -> Path:
        # the verifier's embedding / head are filled at load time, not here
        spec = config.speculators_config
        path, spec.verifier.name_or_path = spec.verifier.name_or_path, None
        model = Eagle3DraftModel(config)
        spec.verifier.name_or_path = path
        result = model.load_state_dict(self.remap_keys(weights), strict=False)
        if result.unexpected_keys:
            log.warning("Unexpected keys in checkpoint: %s", result.unexpected_keys)
        loaded = {k: v for k, v in model.state_dict().items() if k not in result.missing_keys}
        dtype = next((v.dtype for v in weights.values() if v.is_floating_point()), None)
        if dtype is not None:
            loaded = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in loaded.items()}
        model.save_pretrained(str(output_dir), state_dict=loaded)
        return Path(output_dir)
