"""DFlash decoder block: queries come from the noise (draft) tokens only, keys and
values from the projected verifier states followed by the noise tokens
(src/speculators/models/dflash/model_definitions.py:47-207).  K/V of both parts
run as one GEMM over the concatenated rows; per-head q/k RMSNorm; rotary on q with
the noise positions and on k with ``[context positions | noise positions]``."""

from __future__ import annotations

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.layers import MLP, FusedLinear, Linear, RMSNorm, RotaryTable
from speculators_b200.ops import AttnSpec

__all__ = ["DFlashAttention", "DFlashDecoderLayer", "Qwen3DFlashAttention", "Qwen3DFlashDecoderLayer", "apply_rotary_pos_emb"]


class DFlashAttention(nn.Module):
    def __init__(self, config: TransformerLayerConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.nh, self.nkv, self.hd = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        self.rot = config.rotary_dim
        self.scaling = self.hd**-0.5
        self.qkv_proj = FusedLinear(
            config.hidden_size, ["q_proj", "k_proj", "v_proj"], [self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd],
            bias=bool(config.attention_bias),
        ).attach(self, "qkv_proj")
        self.o_proj = Linear(self.nh * self.hd, config.hidden_size, bias=bool(config.attention_bias))
        self.q_norm = RMSNorm(self.hd, config.rms_norm_eps)
        self.k_norm = RMSNorm(self.hd, config.rms_norm_eps)

    def forward(self, noise, target_hidden, noise_positions, all_positions, rotary: RotaryTable, spec: AttnSpec, residual=None):
        nq = noise.shape[0]
        T = target_hidden.shape[0]
        q = self.qkv_proj.forward_parts(noise, 0, 1).view(nq, self.nh, self.hd)
        kv = self.qkv_proj.forward_parts(torch.cat([target_hidden, noise], dim=0), 1, 3)
        k = kv[:, : self.nkv * self.hd].reshape(T + nq, self.nkv, self.hd)
        v = kv[:, self.nkv * self.hd :].view(T + nq, self.nkv, self.hd)
        q = self.q_norm(q).reshape(nq, self.nh * self.hd)
        k = self.k_norm(k).reshape(T + nq, self.nkv * self.hd)
        q = ops.rope_(q, noise_positions, rotary.cos, rotary.sin, self.nh, self.hd, self.rot).view(nq, self.nh, self.hd)
        k = ops.rope_(k, all_positions, rotary.cos, rotary.sin, self.nkv, self.hd, self.rot).view(T + nq, self.nkv, self.hd)
        out = ops.masked_attention(q, k[:T], v[:T], spec, k[T:], v[T:], scale=self.scaling)
        return self.o_proj(out.reshape(nq, self.nh * self.hd), residual=residual)


class DFlashDecoderLayer(nn.Module):
    def __init__(self, config: TransformerLayerConfig, layer_idx: int):
        super().__init__()
        self.self_attn = DFlashAttention(config, layer_idx)
        self.mlp = MLP(config)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, noise, target_hidden, noise_positions, all_positions, rotary, spec):
        noise = self.self_attn(self.input_layernorm(noise), target_hidden, noise_positions, all_positions, rotary, spec, residual=noise)
        return self.mlp(self.post_attention_layernorm(noise), residual=noise)


# names of the reference's Hugging-Face-based classes (src/speculators/models/dflash/model_definitions.py:47,158)
Qwen3DFlashAttention = DFlashAttention
Qwen3DFlashDecoderLayer = DFlashDecoderLayer


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim: int = 1):  # noqa: ARG001
    """Rotate-half rotary embedding of ``q`` and ``k`` ([..., heads, T, hd] with ``cos`` / ``sin``
    [..., T, hd]); when ``q`` is shorter than ``k`` (block queries appended to the context) it
    takes the last ``q_len`` positions (src/speculators/models/dflash/model_definitions.py:29-44).
    The training path applies the same rotation inside ``ops.rope_split``."""
    import torch

    def rotate_half(x):
        a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat((-b, a), dim=-1)

    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    q_len = q.size(-2)
    return q * cos[..., -q_len:, :] + rotate_half(q) * sin[..., -q_len:, :], k * cos + rotate_half(k) * sin
