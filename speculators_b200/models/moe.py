"""Gated-attention + sparse mixture-of-experts decoder block (Qwen3-Next /
Qwen3.5-MoE style) and its MTP variant.

Parameter names follow the Hugging Face modules the reference wraps
(``Qwen3NextDecoderLayer`` via src/speculators/models/mtp/model_definitions.py:159-205
and the fused expert tensors produced by src/speculators/convert/mtp/converter.py:
123-186):

    self_attn.{q,k,v,o}_proj.weight   (q_proj emits [query | gate] per head)
    self_attn.{q,k}_norm.weight       zero-centred RMSNorm over head_dim
    mlp.gate.weight                   router  [E, H]
    mlp.experts.gate_up_proj          [E, 2*I, H]
    mlp.experts.down_proj             [E, H, I]
    mlp.shared_expert.{gate,up,down}_proj.weight,  mlp.shared_expert_gate.weight [1, H]

Routing: softmax over all experts in fp32, top-k, optional renormalisation of the
selected probabilities; output = sum_k p_k * expert_k(x) + sigmoid(shared_gate(x)) *
shared_expert(x).

Expert parallelism (no counterpart in the reference, which only replicates or
FSDP-shards the experts): with ``ep_group`` set, rank ``r`` holds experts
``[r*E/R, (r+1)*E/R)``; tokens are sorted by destination rank, exchanged with
``all_to_all_single`` (dispatch), run through the local experts and sent back
(combine).  ``expert_forward`` is the dense-loop formulation that serves as the
numerical oracle for both paths.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from speculators_b200 import ops
from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.layers import FusedLinear, Linear, RotaryTable
from speculators_b200.models.mtp.model_definitions import _MTPMixin
from speculators_b200.ops import AttnSpec

__all__ = ["GatedAttention", "MoEDecoderLayer", "MoEMTPLayer", "SparseMoeBlock", "ZeroCenteredRMSNorm", "expert_forward"]


class ZeroCenteredRMSNorm(nn.Module):
    """``x / rms(x) * (1 + weight)`` with the weight initialised to zero."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return (xf * (1.0 + self.weight.float())).to(x.dtype)


class GatedAttention(nn.Module):
    def __init__(self, config: TransformerLayerConfig, layer_idx: int):
        super().__init__()
        self.nh, self.nkv, self.hd = config.num_attention_heads, config.num_key_value_heads, config.head_dim
        self.rot = config.rotary_dim
        self.scaling = self.hd**-0.5
        H = config.hidden_size
        bias = bool(config.attention_bias)
        self.q_proj = Linear(H, self.nh * self.hd * 2, bias=bias)
        self.k_proj = Linear(H, self.nkv * self.hd, bias=bias)
        self.v_proj = Linear(H, self.nkv * self.hd, bias=bias)
        self.o_proj = Linear(self.nh * self.hd, H, bias=bias)
        self.q_norm = ZeroCenteredRMSNorm(self.hd, config.rms_norm_eps)
        self.k_norm = ZeroCenteredRMSNorm(self.hd, config.rms_norm_eps)

    def forward(self, x, positions, rotary: RotaryTable, spec: AttnSpec) -> torch.Tensor:
        T = x.shape[0]
        qg = self.q_proj(x).view(T, self.nh, 2 * self.hd)
        q, gate = qg[..., : self.hd], qg[..., self.hd :].reshape(T, self.nh * self.hd)
        q = self.q_norm(q).reshape(T, self.nh * self.hd)
        k = self.k_norm(self.k_proj(x).view(T, self.nkv, self.hd)).reshape(T, self.nkv * self.hd)
        v = self.v_proj(x).view(T, self.nkv, self.hd)
        q = ops.rope_(q.contiguous(), positions, rotary.cos, rotary.sin, self.nh, self.hd, self.rot).view(T, self.nh, self.hd)
        k = ops.rope_(k.contiguous(), positions, rotary.cos, rotary.sin, self.nkv, self.hd, self.rot).view(T, self.nkv, self.hd)
        out = ops.masked_attention(q, k, v, spec, scale=self.scaling).reshape(T, self.nh * self.hd)
        return self.o_proj(out * torch.sigmoid(gate))


class _Experts(nn.Module):
    def __init__(self, num_local: int, hidden: int, inter: int):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(num_local, 2 * inter, hidden).normal_(std=0.02))
        self.down_proj = nn.Parameter(torch.empty(num_local, hidden, inter).normal_(std=0.02))


class _SharedExpert(nn.Module):
    """The always-on expert: a gated MLP with the gate | up projections stored as one weight (one GEMM with the
    activation in its epilogue on CUDA); its state dict keeps the ``gate_proj`` / ``up_proj`` / ``down_proj`` names."""

    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate_up_proj = FusedLinear(hidden, ["gate_proj", "up_proj"], [inter, inter]).attach(self, "gate_up_proj")
        self.down_proj = Linear(inter, hidden)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        hidden = ops.linear_swiglu(x, self.gate_up_proj.weight)
        if hidden is None:
            hidden = ops.swiglu(self.gate_up_proj(x))
        return self.down_proj(hidden)


def expert_forward(x: torch.Tensor, expert_ids: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """Rows of ``x`` through their experts (``expert_ids`` local indices), dense loop."""
    out = torch.zeros_like(x)
    for e in torch.unique(expert_ids).tolist():
        rows = torch.nonzero(expert_ids == e, as_tuple=False).squeeze(-1)
        gu = x[rows] @ gate_up[e].t()
        g, u = gu.chunk(2, dim=-1)
        out[rows] = (F.silu(g) * u) @ down[e].t()
    return out


class _DispatchRows(torch.autograd.Function):
    """``x[order // k]``: every token's row copied to the ``k`` places its experts' sorted order gives it.  The
    backward is a gather through the inverse permutation and a sum over each token's ``k`` copies - no atomics
    (autograd's ``index_add`` for the same gather ran at 250 GB/s on 40960 x 2048 rows)."""

    @staticmethod
    def forward(ctx, x, order, inv, k):
        ctx.save_for_backward(inv)
        ctx.k = k
        return x.index_select(0, torch.div(order, k, rounding_mode="floor"))

    @staticmethod
    def backward(ctx, dxs):
        (inv,) = ctx.saved_tensors
        T = inv.numel() // ctx.k
        return dxs.index_select(0, inv).view(T, ctx.k, dxs.shape[-1]).sum(1), None, None, None


class _CombineRows(torch.autograd.Function):
    """``out[t] = sum_j top_p[t, j] * ys[inv[t * k + j]]``: each token gathers its ``k`` expert outputs from the
    expert-sorted order and forms the weighted sum (instead of scattering weighted rows with atomic adds)."""

    @staticmethod
    def forward(ctx, ys, order, inv, top_p):
        T, k = top_p.shape
        gathered = ys.index_select(0, inv).view(T, k, ys.shape[-1])
        ctx.save_for_backward(ys, order, inv, top_p)
        return (gathered * top_p.unsqueeze(-1)).sum(1)

    @staticmethod
    def backward(ctx, dout):
        ys, order, inv, top_p = ctx.saved_tensors
        T, k = top_p.shape
        H = ys.shape[-1]
        dys = dtop = None
        if ctx.needs_input_grad[0]:
            dys = (dout.unsqueeze(1) * top_p.unsqueeze(-1)).view(T * k, H).index_select(0, order)
        if ctx.needs_input_grad[3]:
            gathered = ys.index_select(0, inv).view(T, k, H)
            dtop = (gathered * dout.unsqueeze(1)).sum(-1).to(top_p.dtype)
        return dys, None, None, dtop


def _grouped_expert_forward(x_sorted: torch.Tensor, counts: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """Rows already sorted by local expert; ``counts[e]`` rows belong to expert ``e``.  bf16 CUDA
    rows with kernel-friendly widths run as grouped launches of the package's tcgen05 GEMM over a
    128-row padded expert order (tile schedule driven by the device-side counts: no host read,
    fixed shapes); ``SB200_MOE_GEMM=library`` or other shapes use the library / the dense loop."""
    if (x_sorted.is_cuda and x_sorted.dtype == torch.bfloat16 and os.environ.get("SB200_MOE_GEMM", "tcgen05") != "library"
            and gate_up.shape[1] % 256 == 0 and gate_up.shape[2] % 256 == 0 and down.shape[2] % 256 == 0 and x_sorted.shape[1] % 8 == 0):
        plan = ops.GroupPlan(counts, x_sorted.shape[0])
        x_pad = plan.pad(x_sorted)
        if ops.grouped_linear_ok(x_pad, gate_up):
            act = ops.swiglu(ops.grouped_linear(x_pad, gate_up, plan))
            return plan.unpad(ops.grouped_linear(act, down, plan))
    grouped = getattr(torch, "_grouped_mm", None)
    if x_sorted.is_cuda and grouped is not None and x_sorted.dtype == torch.bfloat16:
        offs = counts.cumsum(0).to(torch.int32)
        gu = grouped(x_sorted, gate_up.transpose(1, 2), offs=offs)
        g, u = gu.chunk(2, dim=-1)
        return grouped((F.silu(g) * u).contiguous(), down.transpose(1, 2), offs=offs)
    ids = torch.repeat_interleave(torch.arange(counts.numel(), device=x_sorted.device), counts)
    return expert_forward(x_sorted, ids, gate_up, down)


class SparseMoeBlock(nn.Module):
    def __init__(self, config: TransformerLayerConfig, ep_group=None):
        super().__init__()
        H = config.hidden_size
        self.num_experts = int(config.num_experts)
        self.top_k = int(config.num_experts_per_tok)
        self.norm_topk_prob = bool(config.get("norm_topk_prob", True))
        self.ep_group = ep_group
        self.ep_size = dist.get_world_size(ep_group) if ep_group is not None else 1
        self.ep_rank = dist.get_rank(ep_group) if ep_group is not None else 0
        if self.num_experts % self.ep_size:
            raise ValueError(f"num_experts ({self.num_experts}) must be divisible by the expert-parallel size ({self.ep_size})")
        self.num_local = self.num_experts // self.ep_size
        inter = int(config.moe_intermediate_size)
        self.gate = Linear(H, self.num_experts, bias=False)
        self.experts = _Experts(self.num_local, H, inter)
        shared = int(config.get("shared_expert_intermediate_size", 0) or 0)
        self.shared_expert = _SharedExpert(H, shared) if shared > 0 else None
        self.shared_expert_gate = Linear(H, 1, bias=False) if shared > 0 else None
        self._comm = None  # peer-memory exchange buffers, created at the first expert-parallel CUDA call
        if self.ep_size > 1:
            # this rank's experts differ from every other rank's: the training engine keeps them out of
            # its gradient collectives, and checkpoints hold the stack of all ranks' experts
            for p in self.experts.parameters():
                p._sb200_local = True
            self._register_load_state_dict_pre_hook(self._take_own_experts)

    def _take_own_experts(self, state_dict, prefix, *args) -> None:  # noqa: ANN001, ANN002
        """Loading a checkpoint that holds all experts: keep the slice this rank owns."""
        for name in ("gate_up_proj", "down_proj"):
            key = f"{prefix}experts.{name}"
            full = state_dict.get(key)
            if full is not None and full.shape[0] == self.num_experts and self.num_local != self.num_experts:
                state_dict[key] = full[self.ep_rank * self.num_local : (self.ep_rank + 1) * self.num_local]

    def route(self, x: torch.Tensor):
        probs = torch.softmax(self.gate(x).float(), dim=-1)
        top_p, top_e = torch.topk(probs, self.top_k, dim=-1)
        if self.norm_topk_prob:
            top_p = top_p / top_p.sum(dim=-1, keepdim=True)
        return top_p.to(x.dtype), top_e

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        top_p, top_e = self.route(x)
        if self.ep_size > 1 and self._peer_exchange_ok(x):
            out = self._expert_parallel_peer(x, top_p, top_e)
            if self.shared_expert is not None:
                out = out + torch.sigmoid(self.shared_expert_gate(x)) * self.shared_expert(x)
            return out
        flat_e = top_e.reshape(-1)  # [T*k]
        order = torch.argsort(flat_e, stable=True)  # sorted place -> slot (token * k + j)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=x.device)  # slot -> sorted place
        sorted_e = flat_e[order]
        xs = _DispatchRows.apply(x, order, inv, self.top_k)
        if self.ep_size == 1:
            # rows per expert without a host read (``bincount`` sizes its result from the largest id)
            counts = torch.zeros(self.num_experts, dtype=torch.long, device=x.device).index_add_(0, sorted_e, torch.ones_like(sorted_e))
            ys = _grouped_expert_forward(xs, counts, self.experts.gate_up_proj, self.experts.down_proj)
        else:
            ys = self._expert_parallel(xs, sorted_e)
        out = _CombineRows.apply(ys, order, inv, top_p)
        if self.shared_expert is not None:
            out = out + torch.sigmoid(self.shared_expert_gate(x)) * self.shared_expert(x)
        return out

    # ------------------------------------------------------------------ peer-memory exchange
    def _peer_exchange_ok(self, x: torch.Tensor) -> bool:
        """bf16 CUDA activations go through the NVLink peer-memory kernels
        (``parallel/ep_comm.py``); ``SB200_EP_COMM=nccl`` keeps the library all-to-all."""
        return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and os.environ.get("SB200_EP_COMM", "p2p") != "nccl"

    def _ep_comm(self, x: torch.Tensor):
        """Exchange buffers of the group, created (collectively) at the first call.  Capacity:
        ``SB200_EP_CAPACITY_ROWS`` or the worst case of this first call (every slot of every
        rank routed to one rank)."""
        if self._comm is None:
            from speculators_b200.parallel.ep_comm import EpComm

            t_max = torch.tensor([x.shape[0]], device=x.device)
            dist.all_reduce(t_max, op=dist.ReduceOp.MAX, group=self.ep_group)
            rows = int(os.environ.get("SB200_EP_CAPACITY_ROWS", 0)) or self.ep_size * int(t_max.item()) * self.top_k
            self._comm = EpComm(self.ep_group, x.shape[1], rows, x.device)
            self._comm.connect()
        return self._comm

    def _expert_parallel_peer(self, x: torch.Tensor, top_p: torch.Tensor, top_e: torch.Tensor) -> torch.Tensor:
        """Dispatch, local experts, weighted combine with the rows moved by peer-memory
        kernels; only the token counts go through the process group."""
        from speculators_b200.parallel.ep_comm import build_plan, ep_combine, ep_dispatch

        comm = self._ep_comm(x)
        counts = torch.bincount(top_e.reshape(-1), minlength=self.num_experts)
        counts_all = torch.empty(self.ep_size, self.num_experts, dtype=counts.dtype, device=x.device)
        dist.all_gather_into_tensor(counts_all, counts, group=self.ep_group)
        plan = build_plan(top_e, counts_all, self.ep_rank, self.num_local)
        if plan.max_recv > comm.capacity:
            raise RuntimeError(f"expert-parallel receive buffer too small: a rank receives {plan.max_recv} rows, capacity is "
                               f"{comm.capacity}; set SB200_EP_CAPACITY_ROWS")
        plan.parity = comm.next_parity()
        recv_x = ep_dispatch(x, comm, plan)
        ys = _grouped_expert_forward(recv_x, plan.local_counts, self.experts.gate_up_proj, self.experts.down_proj)
        return ep_combine(ys, top_p, comm, plan)

    def _expert_parallel(self, xs: torch.Tensor, sorted_e: torch.Tensor) -> torch.Tensor:
        """Dispatch (all-to-all), local experts, combine (all-to-all).  Rows arrive
        already grouped by destination rank because experts are sorted."""
        R, group = self.ep_size, self.ep_group
        send_counts = torch.bincount(sorted_e // self.num_local, minlength=R)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        send, recv = send_counts.tolist(), recv_counts.tolist()
        recv_x = _AllToAll.apply(xs, recv, send, group)
        recv_e = torch.empty(sum(recv), dtype=sorted_e.dtype, device=xs.device)
        dist.all_to_all_single(recv_e, sorted_e.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        local_e = recv_e - self.ep_rank * self.num_local
        order = torch.argsort(local_e, stable=True)
        counts = torch.bincount(local_e, minlength=self.num_local)
        ys_local = _grouped_expert_forward(recv_x[order], counts, self.experts.gate_up_proj, self.experts.down_proj)
        back = torch.empty_like(ys_local)
        back[order] = ys_local
        return _AllToAll.apply(back, send, recv, group)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.splits = (out_splits, in_splits)
        ctx.group = group
        out = torch.empty((sum(out_splits), *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, dout):
        out_splits, in_splits = ctx.splits
        dx = torch.empty((sum(in_splits), *dout.shape[1:]), dtype=dout.dtype, device=dout.device)
        dist.all_to_all_single(dx, dout.contiguous(), output_split_sizes=in_splits, input_split_sizes=out_splits, group=ctx.group)
        return dx, None, None, None


class MoEDecoderLayer(nn.Module):
    def __init__(self, config: TransformerLayerConfig, layer_idx: int, ep_group=None):
        super().__init__()
        H, eps = config.hidden_size, config.rms_norm_eps
        self.self_attn = GatedAttention(config, layer_idx)
        self.mlp = SparseMoeBlock(config, ep_group=ep_group)
        self.input_layernorm = ZeroCenteredRMSNorm(H, eps)
        self.post_attention_layernorm = ZeroCenteredRMSNorm(H, eps)

    def forward(self, x, positions, rotary, spec) -> torch.Tensor:
        x = x + self.self_attn(self.input_layernorm(x), positions, rotary, spec)
        return x + self.mlp(self.post_attention_layernorm(x))


class MoEMTPLayer(_MTPMixin, MoEDecoderLayer):
    """``ep_group``: process group over which the experts are split (expert parallelism); ``None``
    keeps all experts on every rank."""

    def __init__(self, config: TransformerLayerConfig, layer_idx: int = 0, ep_group=None):
        MoEDecoderLayer.__init__(self, config, layer_idx, ep_group=ep_group)
        self._setup_mtp_modules(config, norm_cls=ZeroCenteredRMSNorm)

    def forward(self, hidden_states, token_embeddings, positions, rotary, spec):
        x = self.combine(hidden_states, token_embeddings)
        return self.final_layernorm(MoEDecoderLayer.forward(self, x, positions, rotary, spec))
