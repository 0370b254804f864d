"""Decoder building blocks owned by this framework.

The reference assembles its drafts from Hugging Face ``LlamaDecoderLayer`` /
``Qwen3DecoderLayer`` classes (src/speculators/models/base_components.py:39-100).
Here the blocks are written against ``speculators_b200.ops`` so that on a B200
every hot step is one of the package's own kernels, while the parameter *names*
in ``state_dict()`` stay the Hugging Face ones (``self_attn.q_proj.weight``,
``mlp.gate_proj.weight`` ...), which is what the checkpoint format and vLLM
expect.

Projections that share an input are stored fused (q|k|v and gate|up) so each
runs as a single GEMM; ``FusedLinear`` splits / merges them at the
``state_dict`` boundary.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from speculators_b200 import ops
from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.ops import AttnSpec

__all__ = [
    "Attention",
    "DecoderLayer",
    "FusedLinear",
    "Linear",
    "MLP",
    "RMSNorm",
    "RotaryTable",
]


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.variance_epsilon)

    def extra_repr(self) -> str:
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


def _init_linear_(weight: torch.Tensor, std: float = 0.02) -> None:
    with torch.no_grad():
        weight.normal_(mean=0.0, std=std)


class Linear(nn.Module):
    """Bias-optional linear layer; weight ``[out, in]`` like ``nn.Linear``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, std: float = 0.02):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        # tensor parallelism (inference): ``row_parallel(x, weight, residual) -> sum over the ranks'
        # partial products + residual`` replaces the local product of a layer whose input is split
        self.row_parallel = None
        _init_linear_(self.weight, std)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.row_parallel is not None and self.bias is None:
            return self.row_parallel(x, self.weight, residual)
        return ops.linear(x, self.weight, self.bias, residual=residual)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class FusedLinear(nn.Module):
    """Several projections of the same input stored as one ``[sum(out), in]`` weight.

    ``names``/``sizes`` describe the parts.  ``state_dict`` exposes them as
    ``<prefix><name>.weight`` (and ``.bias``) exactly as separate ``nn.Linear``
    modules would, and loading accepts the split form, so checkpoints are
    indistinguishable from the unfused layout.
    """

    def __init__(self, in_features: int, names: list[str], sizes: list[int], bias: bool = False):
        super().__init__()
        self.in_features = in_features
        self.names, self.sizes = list(names), list(sizes)
        self.weight = nn.Parameter(torch.empty(sum(sizes), in_features))
        self.bias = nn.Parameter(torch.zeros(sum(sizes))) if bias else None
        _init_linear_(self.weight)
        self._register_state_dict_hook(FusedLinear._split_on_save)

    def attach(self, parent: nn.Module, attr: str) -> "FusedLinear":
        """Register the load-time merge on ``parent`` (the module that holds this
        layer as attribute ``attr``).  ``load_state_dict`` hands a child only the keys
        under the child's own prefix, so the split names ``<parent>.<part>.weight``
        are visible to the parent alone."""

        def merge(state_dict, prefix, *args):  # noqa: ANN001, ANN002
            for kind in ("weight", "bias"):
                keys = [f"{prefix}{name}.{kind}" for name in self.names]
                if all(k in state_dict for k in keys):
                    state_dict[f"{prefix}{attr}.{kind}"] = torch.cat([state_dict.pop(k) for k in keys], dim=0)

        parent._register_load_state_dict_pre_hook(merge)
        return self

    def offsets(self) -> list[int]:
        out, acc = [], 0
        for s in self.sizes:
            out.append(acc)
            acc += s
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)

    def forward_parts(self, x: torch.Tensor, first: int, last: int) -> torch.Tensor:
        """Apply only parts ``first .. last-1`` (row slice of the fused weight)."""
        offs = self.offsets() + [sum(self.sizes)]
        return ops.linear(x, self.weight, self.bias, rows=(offs[first], offs[last]))

    # the hooks see keys like "<prefix>weight"; the parent prefix (without this
    # module's own attribute name) is where the split names live.
    @staticmethod
    def _parent_prefix(prefix: str) -> str:
        trimmed = prefix[:-1] if prefix.endswith(".") else prefix
        return trimmed.rsplit(".", 1)[0] + "." if "." in trimmed else ""

    @staticmethod
    def _split_on_save(module, state_dict, prefix, local_metadata):  # noqa: ANN001, ARG004
        parent = FusedLinear._parent_prefix(prefix)
        for kind in ("weight", "bias"):
            fused = state_dict.pop(prefix + kind, None)
            if fused is None:
                continue
            for name, off, size in zip(module.names, module.offsets(), module.sizes):
                state_dict[f"{parent}{name}.{kind}"] = fused[off : off + size]
        return state_dict

    def extra_repr(self) -> str:
        parts = ", ".join(f"{n}:{s}" for n, s in zip(self.names, self.sizes))
        return f"in={self.in_features}, parts=[{parts}], bias={self.bias is not None}"


class RotaryTable(nn.Module):
    """fp32 cos/sin tables ``[max_pos, rot/2]`` (non-persistent buffers).

    Supports the ``default``, ``linear`` and ``llama3`` frequency schedules of
    Hugging Face ``rope_scaling`` / ``rope_parameters`` dicts.
    """

    def __init__(self, config: TransformerLayerConfig, max_positions: int | None = None):
        super().__init__()
        self.rot = config.rotary_dim
        self.head_dim = config.head_dim
        self.max_positions = int(max_positions or min(int(config.max_position_embeddings), 1 << 17))
        self.theta = float(config.rope_theta)
        scaling = config.get("rope_scaling") or config.get("rope_parameters") or {}
        if "sliding_attention" in scaling:
            scaling = scaling["sliding_attention"]
        self.scaling = dict(scaling) if isinstance(scaling, dict) else {}
        self.register_buffer("cos", torch.empty(0), persistent=False)
        self.register_buffer("sin", torch.empty(0), persistent=False)
        self._build(self.max_positions)

    def _inv_freq(self) -> torch.Tensor:
        rot = self.rot
        inv = 1.0 / (self.theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))
        kind = self.scaling.get("rope_type", self.scaling.get("type", "default"))
        if kind == "linear":
            inv = inv / float(self.scaling.get("factor", 1.0))
        elif kind == "llama3":
            factor = float(self.scaling.get("factor", 8.0))
            lo = float(self.scaling.get("low_freq_factor", 1.0))
            hi = float(self.scaling.get("high_freq_factor", 4.0))
            orig = float(self.scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv
            smooth = ((orig / wavelen) - lo) / (hi - lo)
            blended = (1 - smooth) * inv / factor + smooth * inv
            inv = torch.where(wavelen > orig / lo, inv / factor, torch.where(wavelen < orig / hi, inv, blended))
        return inv

    def _build(self, n: int) -> None:
        device = self.cos.device
        ang = torch.outer(torch.arange(n, dtype=torch.float64), self._inv_freq())
        self.cos = ang.cos().float().to(device).contiguous()
        self.sin = ang.sin().float().to(device).contiguous()
        self.max_positions = n

    def _apply(self, fn, recurse=True):  # noqa: ANN001
        """Keep the tables in fp32 whatever dtype the owning model is cast to."""
        super()._apply(fn, recurse)
        if self.cos.dtype != torch.float32:
            self.cos, self.sin = self.cos.float(), self.sin.float()
            self._build(self.max_positions)
        return self

    def ensure(self, max_pos: int) -> None:
        """Grow the tables (host side, outside any captured region) to cover ``max_pos``."""
        if max_pos >= self.max_positions:
            self._build(int(max_pos * 2))


class Attention(nn.Module):
    """Grouped-query self-attention over an ``AttnSpec`` mask.

    ``input_size`` differs from ``hidden_size`` only for the EAGLE-3 first layer,
    whose q/k/v projections read ``cat([embeds, hidden])`` (2H).
    """

    def __init__(self, config: TransformerLayerConfig, layer_idx: int, input_size: int | None = None, qk_norm: bool | None = None):
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.nh, self.nkv, self.hd = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        self.rot = config.rotary_dim
        self.scaling = self.hd**-0.5
        in_size = input_size or config.hidden_size
        self.qkv_proj = FusedLinear(
            in_size, ["q_proj", "k_proj", "v_proj"],
            [self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd], bias=bool(config.attention_bias),
        ).attach(self, "qkv_proj")
        self.o_proj = Linear(self.nh * self.hd, config.hidden_size, bias=bool(config.attention_bias))
        use_qk_norm = config.model_type.startswith("qwen3") if qk_norm is None else qk_norm
        self.q_norm = RMSNorm(self.hd, config.rms_norm_eps) if use_qk_norm else None
        self.k_norm = RMSNorm(self.hd, config.rms_norm_eps) if use_qk_norm else None

    def project_qkv(self, x: torch.Tensor, positions: torch.Tensor, rotary: RotaryTable):
        """x [T, in] -> (q [T, nh, hd], k [T, nkv, hd], v [T, nkv, hd]) with per-head
        norms (if any) and rotary embedding applied.  The three results are views
        of one fused projection buffer."""
        T = x.shape[0]
        nq, nk = self.nh * self.hd, self.nkv * self.hd
        qkv = self.qkv_proj(x)
        if self.q_norm is not None:
            q = self.q_norm(qkv[:, :nq].reshape(T, self.nh, self.hd))
            k = self.k_norm(qkv[:, nq : nq + nk].reshape(T, self.nkv, self.hd))
            qk = torch.cat([q.reshape(T, nq), k.reshape(T, nk)], dim=-1)
            qk = ops.rope_(qk, positions, rotary.cos, rotary.sin, self.nh + self.nkv, self.hd, self.rot)
            q, k = qk[:, :nq], qk[:, nq:]
            v = qkv[:, nq + nk :]
        else:
            q, k, v = ops.rope_split(qkv, positions, rotary.cos, rotary.sin, self.nh + self.nkv, self.hd, self.rot, nq, nk)
        return q.view(T, self.nh, self.hd), k.view(T, self.nkv, self.hd), v.view(T, self.nkv, self.hd)

    def forward(self, x, positions, rotary, spec: AttnSpec, past: list | None = None, ctx_len: int | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        """``past`` (EAGLE-3 TTT): list of (k, v) of earlier passes over the same
        positions.  Entry 0 is the context the interval part of ``spec`` indexes;
        later entries and this pass's own keys are reachable through
        ``spec.extra_idx`` (row ``(j-1)*T + i`` = key ``i`` of pass ``j``).

        ``ctx_len`` (P-EAGLE): the first ``ctx_len`` rows of this pass are the
        interval-addressed context, the remaining rows are the extra keys."""
        T = x.shape[0]
        q, k, v = self.project_qkv(x, positions, rotary)
        if ctx_len is not None and ctx_len < T:
            out = ops.masked_attention(q, k[:ctx_len], v[:ctx_len], spec, k[ctx_len:], v[ctx_len:], scale=self.scaling)
        elif past is None:
            out = ops.masked_attention(q, k, v, spec, scale=self.scaling)
        else:
            past.append((k, v))
            k_ctx, v_ctx = past[0]
            if len(past) > 1:
                k_ext = torch.cat([kv[0] for kv in past[1:]], dim=0)
                v_ext = torch.cat([kv[1] for kv in past[1:]], dim=0)
                out = ops.masked_attention(q, k_ctx, v_ctx, spec, k_ext, v_ext, scale=self.scaling)
            else:
                out = ops.masked_attention(q, k_ctx, v_ctx, spec, scale=self.scaling)
        return self.o_proj(out.reshape(T, self.nh * self.hd), residual=residual)


_GATE_ACTIVATIONS = {
    "gelu": lambda g: torch.nn.functional.gelu(g),
    "gelu_new": lambda g: torch.nn.functional.gelu(g, approximate="tanh"),
    "gelu_pytorch_tanh": lambda g: torch.nn.functional.gelu(g, approximate="tanh"),
    "relu": torch.relu,
}


class MLP(nn.Module):
    """Gated MLP ``down(act(gate(x)) * up(x))``.  SiLU (every supported verifier family's default)
    runs on the fused SwiGLU kernel; the other activations the reference accepts through
    ``--draft-hidden-act`` (GELU variants, ReLU) use the element-wise PyTorch formulation."""

    def __init__(self, config: TransformerLayerConfig, intermediate_size: int | None = None):
        super().__init__()
        inter = intermediate_size or config.intermediate_size
        self.hidden_act = str(config.hidden_act)
        if self.hidden_act not in ("silu", "swish") and self.hidden_act not in _GATE_ACTIVATIONS:
            raise ValueError(f"hidden_act={config.hidden_act!r} is not supported; choose one of {['silu', *sorted(_GATE_ACTIVATIONS)]}")
        self.gate_up_proj = FusedLinear(config.hidden_size, ["gate_proj", "up_proj"], [inter, inter], bias=bool(config.mlp_bias)).attach(self, "gate_up_proj")
        self.down_proj = Linear(inter, config.hidden_size, bias=bool(config.mlp_bias))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        silu = self.hidden_act in ("silu", "swish")
        if silu and self.gate_up_proj.bias is None:
            hidden = ops.linear_swiglu(x, self.gate_up_proj.weight)  # activation in the GEMM's epilogue
            if hidden is not None:
                return self.down_proj(hidden, residual=residual)
        gate_up = self.gate_up_proj(x)
        if silu:
            hidden = ops.swiglu(gate_up)
        else:
            gate, up = gate_up.chunk(2, dim=-1)
            hidden = _GATE_ACTIVATIONS[self.hidden_act](gate) * up
        return self.down_proj(hidden, residual=residual)


class DecoderLayer(nn.Module):
    """Pre-norm decoder block (Llama / Qwen3 layout)."""

    def __init__(self, config: TransformerLayerConfig, layer_idx: int):
        super().__init__()
        self.self_attn = Attention(config, layer_idx)
        self.mlp = MLP(config)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, x, positions, rotary, spec, past=None, ctx_len=None) -> torch.Tensor:
        x = self.self_attn(self.input_layernorm(x), positions, rotary, spec, past, ctx_len, residual=x)
        return self.mlp(self.post_attention_layernorm(x), residual=x)
