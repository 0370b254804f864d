"""External DFlash checkpoint -> speculators format
(src/speculators/convert/dflash/converter.py:48-251): the decoder body is copied
(fused ``qkv_proj`` split into q/k/v, ``g_proj`` / ``aux_hidden_norms`` dropped,
``fc.weight`` sliced if the source used more aux layers), the verifier fills the
embedding / LM head / final norm, target layer ids are shifted by one to the
convention used here."""

from __future__ import annotations

import logging
from pathlib import Path

import torch

from speculators_b200.config import SpeculatorsConfig, VerifierConfig
from speculators_b200.convert.utils import ensure_checkpoint_is_local, load_checkpoint_config, load_checkpoint_weights
from speculators_b200.layer_config import read_config_json
from speculators_b200.models.dflash import DFlashDraftModel, DFlashSpeculatorConfig
from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

log = logging.getLogger("speculators")

__all__ = ["DFlashConverter"]

_NON_DECODER_KEYS = frozenset({"architectures", "auto_map", "block_size", "dflash_config", "num_target_layers"})
_VERIFIER_FILLED = frozenset({"embed_tokens.weight", "lm_head.weight", "verifier_lm_head.weight", "verifier_norm.weight", "t2d", "d2t"})


class DFlashConverter:
    def convert(self, input_path, output_path, base_model: str, validate: bool = True, aux_hidden_state_layer_ids: list[int] | None = None, cache_dir=None) -> None:
        local = ensure_checkpoint_is_local(input_path, cache_dir)
        config = self._build_config(load_checkpoint_config(local), base_model, aux_hidden_state_layer_ids)
        saved = self._save(config, load_checkpoint_weights(local), output_path)
        log.info("Saved to: %s", saved)
        if validate:
            model = DFlashDraftModel.from_pretrained(str(saved))
            for name in ("fc.weight", "lm_head.weight", "embed_tokens.weight"):
                if torch.isnan(model.state_dict()[name]).any():
                    raise ValueError(f"Converted checkpoint has NaN in {name}")

    def _build_config(self, source: dict, base_model: str, aux_ids: list[int] | None) -> DFlashSpeculatorConfig:
        extra = source.get("dflash_config", {})
        block_size = source.get("block_size") or extra.get("block_size")
        if block_size is None:
            raise ValueError("Checkpoint config has no `block_size` (checked both top-level and `dflash_config`)")
        decoder = {k: v for k, v in source.items() if k not in _NON_DECODER_KEYS}
        verifier = read_config_json(base_model)
        if decoder.get("hidden_size") and verifier.get("hidden_size") and decoder["hidden_size"] != verifier["hidden_size"]:
            raise ValueError(
                f"Architecture mismatch: source DFlash checkpoint has hidden_size={decoder['hidden_size']} but base_model "
                f"'{base_model}' has hidden_size={verifier['hidden_size']}. Dimensions must match."
            )
        if aux_ids is None:
            target_ids = extra.get("target_layer_ids")
            if target_ids is None:
                raise ValueError("Checkpoint config has no `dflash_config.target_layer_ids`; pass `aux_hidden_state_layer_ids` explicitly.")
            aux_ids = [i + 1 for i in target_ids if i + 1 != verifier["num_hidden_layers"]]
        return DFlashSpeculatorConfig(
            transformer_layer_config=decoder, draft_vocab_size=decoder["vocab_size"], block_size=block_size,
            aux_hidden_state_layer_ids=aux_ids, mask_token_id=extra.get("mask_token_id"),
            speculators_config=SpeculatorsConfig(
                algorithm="dflash", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=block_size - 1)],
                default_proposal_method="greedy", verifier=VerifierConfig(name_or_path=base_model, architectures=verifier.get("architectures", [])),
            ),
        )

    @staticmethod
    def remap_weights(weights: dict, fc_in_features: int) -> dict:
        out, dropped = {}, []
        for key, tensor in weights.items():
            if ".g_proj." in key or key.startswith("aux_hidden_norms."):
                dropped.append(key)
            elif key == "fc.weight" and tensor.shape[1] > fc_in_features:
                out[key] = tensor[:, :fc_in_features]
            else:
                out[key] = tensor  # a fused qkv_proj loads as is: the decoder here stores q|k|v fused
        if dropped:
            log.info("Dropped %d incompatible keys: %s", len(dropped), dropped)
        return out

    def _save(self, config, weights, output_path) -> Path:
        model = DFlashDraftModel(config)
        body = self.remap_weights({k: v for k, v in weights.items() if k not in ("t2d", "d2t")}, model.fc.in_features)
        for key in list(body):  # "<x>.qkv_proj.weight" alongside split keys would be ambiguous
            if "qkv_proj" in key and key.replace("qkv_proj", "q_proj") in body:
                raise ValueError(f"Checkpoint contains both fused qkv_proj and separate projection keys near {key}")
        result = model.load_state_dict(body, strict=False)
        if result.unexpected_keys:
            raise ValueError(f"Unexpected keys in checkpoint -- the structure does not match DFlashDraftModel. Unexpected keys: {result.unexpected_keys}")
        critical = [k for k in result.missing_keys if k not in _VERIFIER_FILLED]
        if critical:
            raise ValueError(f"Draft weights missing after load: {critical}")
        model.load_verifier_weights()
        model.to(dtype=next(iter(body.values())).dtype)
        model.save_pretrained(str(output_path))
        return Path(output_path)
