"""Extraction of a verifier's native MTP head (``mtp.*`` tensors) into the MTP
speculator layout (src/speculators/convert/mtp/converter.py:35-316): key remap
(``mtp.fc`` -> ``input_proj``, ``mtp.norm`` -> ``final_layernorm``,
``mtp.pre_fc_norm_hidden`` / ``_embedding`` -> ``hidden_layernorm`` /
``token_layernorm``, ``mtp.layers.0.`` -> ``mtp_layers.0.``) and fusing of
per-expert MoE weights into the packed 3-D ``experts.gate_up_proj`` /
``experts.down_proj`` tensors.  Only shards that hold ``mtp.*`` keys are opened.
"""

from __future__ import annotations

import json
import logging
import re
from pathlib import Path

import torch
from safetensors import safe_open

from speculators_b200.convert.utils import ensure_checkpoint_is_local, load_checkpoint_config
from speculators_b200.utils.loading import list_checkpoint_keys

log = logging.getLogger("speculators")

__all__ = ["MTP_EXACT_REMAP", "MTP_PREFIX_REMAP", "MTPConverter"]

MTP_EXACT_REMAP = {"mtp.fc.weight": "mtp_layers.0.input_proj.weight", "mtp.norm.weight": "mtp_layers.0.final_layernorm.weight"}
MTP_PREFIX_REMAP = [
    ("mtp.pre_fc_norm_hidden.", "mtp_layers.0.hidden_layernorm."),
    ("mtp.pre_fc_norm_embedding.", "mtp_layers.0.token_layernorm."),
    ("mtp.layers.0.", "mtp_layers.0."),
]
_EXPERT = re.compile(r"^(.+\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")


class MTPConverter:
    @staticmethod
    def remap_key(key: str) -> str:
        if key in MTP_EXACT_REMAP:
            return MTP_EXACT_REMAP[key]
        for src, dst in MTP_PREFIX_REMAP:
            if key.startswith(src):
                return dst + key[len(src):]
        return key

    _remap_key = remap_key  # the reference's spelling of the two helpers

    @staticmethod
    def fuse_moe_experts(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        groups: dict[str, dict[int, dict[str, torch.Tensor]]] = {}
        rest: dict[str, torch.Tensor] = {}
        for key, tensor in weights.items():
            m = _EXPERT.match(key)
            if m:
                groups.setdefault(m.group(1), {}).setdefault(int(m.group(2)), {})[m.group(3)] = tensor
            else:
                rest[key] = tensor
        for prefix, by_idx in groups.items():
            n = max(by_idx) + 1
            if set(by_idx) != set(range(n)):
                raise ValueError(f"Non-contiguous expert indices at {prefix}: found {sorted(by_idx)}, expected 0..{n - 1}")
            for i in range(n):
                for proj in ("gate_proj", "up_proj", "down_proj"):
                    if proj not in by_idx[i]:
                        raise ValueError(f"Expert {i} at {prefix} missing {proj} weight")
            rest[f"{prefix}.gate_up_proj"] = torch.stack([torch.cat([by_idx[i]["gate_proj"], by_idx[i]["up_proj"]], dim=0) for i in range(n)])
            rest[f"{prefix}.down_proj"] = torch.stack([by_idx[i]["down_proj"] for i in range(n)])
        return rest

    _fuse_moe_experts = fuse_moe_experts

    def convert_to_state_dict(self, input_path, cache_dir=None) -> dict[str, torch.Tensor]:
        local = ensure_checkpoint_is_local(input_path, cache_dir)
        keys = list_checkpoint_keys(local)
        wanted = {k for k in keys if k.startswith("mtp.")}
        if not wanted:
            raise ValueError("No keys with prefix 'mtp.' found. This converter requires checkpoints with native MTP layers (e.g. Qwen3-Next, Qwen3.5, Qwen3.5-MoE).")
        index = local / "model.safetensors.index.json"
        by_shard: dict[str, list[str]] = {}
        if index.exists():
            wmap = json.loads(index.read_text())["weight_map"]
            for key in wanted:
                by_shard.setdefault(wmap[key], []).append(key)
        else:
            by_shard["model.safetensors"] = sorted(wanted)
        out: dict[str, torch.Tensor] = {}
        for shard, names in by_shard.items():
            with safe_open(str(local / shard), framework="pt") as fh:
                for key in names:
                    out[self.remap_key(key)] = fh.get_tensor(key)
        out = self.fuse_moe_experts(out)
        log.info("Extracted %d MTP weight tensors from %s", len(out), input_path)
        return out

    def convert(self, input_path, output_path, base_model: str, num_speculative_steps: int = 3, validate: bool = True, cache_dir=None) -> None:
        from speculators_b200.config import SpeculatorsConfig, VerifierConfig
        from speculators_b200.layer_config import read_config_json
        from speculators_b200.models.mtp import MTPDraftModel, MTPSpeculatorConfig
        from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

        weights = self.convert_to_state_dict(input_path, cache_dir)
        source = load_checkpoint_config(ensure_checkpoint_is_local(input_path, cache_dir))
        source = source.get("text_config", source)
        verifier = read_config_json(base_model)
        v_hidden = verifier.get("text_config", verifier).get("hidden_size")
        if source.get("hidden_size") and v_hidden and source["hidden_size"] != v_hidden:
            raise ValueError(
                f"Architecture mismatch: source MTP checkpoint has hidden_size={source['hidden_size']} but base_model "
                f"'{base_model}' has hidden_size={v_hidden}. Dimensions must match."
            )
        config = MTPSpeculatorConfig(
            transformer_layer_config=source,
            speculators_config=SpeculatorsConfig(
                algorithm="mtp", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=num_speculative_steps)],
                default_proposal_method="greedy", verifier=VerifierConfig(name_or_path=base_model, architectures=verifier.get("architectures", [])),
            ),
        )
        model = MTPDraftModel(config)
        result = model.load_state_dict(weights, strict=False)
        if result.unexpected_keys:
            raise ValueError(f"Unexpected keys in extracted weights -- the checkpoint structure does not match the model architecture. Unexpected keys: {result.unexpected_keys}")
        critical = [k for k in result.missing_keys if k.startswith("mtp_layers.")]
        if critical:
            raise ValueError(f"Critical MTP layer weights missing after extraction. Missing keys: {critical}")
        dtype = next((t.dtype for t in weights.values() if t.is_floating_point()), None)
        state = {k: v for k, v in model.state_dict().items() if k.startswith("mtp_layers.")}
        if dtype is not None:
            state = {k: v.to(dtype) for k, v in state.items()}
        model.save_pretrained(str(output_path), state_dict=state)
        log.info("Saved to: %s", output_path)
        if validate:
            MTPDraftModel.from_pretrained(str(output_path))
