"""Verifier forward pass that yields the hidden states a draft is trained on.

The reference never runs the verifier itself: a vLLM server does, and ships
``[seq, layers, H]`` hidden states back through ``hs_connectors``
(scripts/launch_vllm.py:129-163; src/speculators/train/data.py:294-304 splits them
into the concatenated aux states and the last layer's output).  This module is
the in-framework producer for dense Llama / Qwen3 verifiers: it returns

* ``hidden_states``  ``[T, len(layer_ids) * H]``: outputs of the requested decoder
  layers, concatenated along the feature dim in the order given, and
* ``verifier_last_hidden_states`` ``[T, H]``: output of the last decoder layer
  (before the final norm; the draft applies ``verifier_norm`` itself).

Two weight sources: a real checkpoint directory (layer weights are read shard by
shard) or seeded random initialisation generated layer by layer, so a
multi-billion-parameter random verifier never has to be resident at once.
"""

from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.eagle3.attention import causal_document_interval
from speculators_b200.models.layers import DecoderLayer, RotaryTable
from speculators_b200.ops import AttnSpec

__all__ = ["RandomVerifier", "write_random_verifier_stub"]


def _seeded(shape, std: float, seed: int, device, dtype) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


class RandomVerifier:
    """Random-init dense decoder evaluated one layer at a time.

    Layer ``i`` is materialised from ``seed * 1000 + i``, used and dropped, which
    bounds memory to one layer regardless of depth.  ``embed_tokens`` / ``lm_head``
    / ``norm`` use fixed sub-seeds so that ``write_random_verifier_stub`` saves
    exactly the tensors this forward used.
    """

    def __init__(self, config: TransformerLayerConfig | dict, seed: int = 0, device="cpu", dtype=torch.float32):
        self.cfg = TransformerLayerConfig.from_any(config)
        self.seed, self.device, self.dtype = seed, torch.device(device), dtype
        self.rotary = RotaryTable(self.cfg).to(self.device)

    def embed_weight(self) -> torch.Tensor:
        return _seeded((self.cfg.vocab_size, self.cfg.hidden_size), 0.02, self.seed * 1000 + 900, self.device, self.dtype)

    def lm_head_weight(self) -> torch.Tensor:
        return _seeded((self.cfg.vocab_size, self.cfg.hidden_size), 0.02, self.seed * 1000 + 901, self.device, self.dtype)

    def norm_weight(self) -> torch.Tensor:
        return torch.ones(self.cfg.hidden_size, device=self.device, dtype=self.dtype)

    def _layer(self, idx: int) -> DecoderLayer:
        layer = DecoderLayer(self.cfg, idx)
        with torch.no_grad():
            for j, p in enumerate(layer.parameters()):
                if p.ndim == 2:
                    p.data = _seeded(tuple(p.shape), 0.02, (self.seed * 1000 + idx) * 64 + j, self.device, self.dtype)
                else:
                    p.data = p.data.to(device=self.device, dtype=self.dtype)
        return layer

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, layer_ids: list[int], document_ids: torch.Tensor | None = None, position_ids: torch.Tensor | None = None):
        ids = input_ids.reshape(-1).to(self.device)
        T = ids.shape[0]
        doc = document_ids.reshape(-1).to(self.device) if document_ids is not None else torch.zeros(T, dtype=torch.long, device=self.device)
        pos = position_ids.reshape(-1).to(self.device) if position_ids is not None else torch.arange(T, device=self.device)
        lo, hi = causal_document_interval(doc)
        spec = AttnSpec(lo=lo, hi=hi)
        h = torch.nn.functional.embedding(ids, self.embed_weight())
        captured: dict[int, torch.Tensor] = {}
        for i in range(int(self.cfg.num_hidden_layers)):
            layer = self._layer(i)
            h = layer(h, pos, self.rotary, spec)
            if i in layer_ids:
                captured[i] = h
            del layer
        aux = torch.cat([captured[i] for i in layer_ids], dim=-1)
        return {"hidden_states": aux, "verifier_last_hidden_states": h}


def write_random_verifier_stub(path: str, config: dict, seed: int = 0, dtype=torch.bfloat16, device="cpu") -> str:
    """Write the part of a verifier checkpoint a draft needs: ``config.json`` and a
    ``model.safetensors`` holding ``model.embed_tokens.weight``, ``lm_head.weight``
    and ``model.norm.weight`` of the ``RandomVerifier`` with the same seed."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(config, fh, indent=2)
    rv = RandomVerifier(config, seed=seed, device=device, dtype=dtype)
    save_file(
        {
            "model.embed_tokens.weight": rv.embed_weight().cpu().contiguous(),
            "lm_head.weight": rv.lm_head_weight().cpu().contiguous(),
            "model.norm.weight": rv.norm_weight().cpu().contiguous(),
        },
        os.path.join(path, "model.safetensors"),
        metadata={"format": "pt"},
    )
    return path
