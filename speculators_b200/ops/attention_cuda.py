"""CUDA path of ``masked_attention``: autograd wrapper around the sm_100a kernels
(head dims 64, 128 and 256).  Other head dims use the dense formulation.

Forward and backward at head dim 128 run on the tcgen05 tensor cores
(``csrc/attention_tc.cu``, ``csrc/attention_bwd_tc.cu``: TMA tiles, TMEM accumulators,
probability tiles handed to the next product through TMEM); ``FWD_IMPL`` / ``BWD_IMPL`` =
``"mma"`` (or ``SB200_ATTN_FWD=mma`` / ``SB200_ATTN_BWD=mma``) select the ``mma.sync``
kernels of ``csrc/attention.cu``, which also serve head dims 64 and 256 (256: the gated
full-attention heads of Qwen3-Next style MTP layers)."""

from __future__ import annotations

import os

import torch

from speculators_b200.ops import _ext
from speculators_b200.ops.attention import AttnSpec, masked_attention_reference

_SUPPORTED_HEAD_DIMS = (64, 128, 256)
FWD_IMPL = os.environ.get("SB200_ATTN_FWD", "tc")
BWD_IMPL = os.environ.get("SB200_ATTN_BWD", "tc")
BLOCK_EXTRAS = os.environ.get("SB200_ATTN_BLOCK_EXTRAS", "1") != "0"  # 0: anchored blocks through the per-row extra-key path


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """[T, heads, hd] with contiguous heads and 16-byte aligned rows (views into a
    fused projection buffer qualify as they are)."""
    hd = t.shape[2]
    if t.stride(2) == 1 and t.stride(1) == hd and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _MaskedAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, lo, hi, k_ext, v_ext, ext_idx, scale, ext_block, ext_causal):
        q, k, v = _rows_ok(q), _rows_ok(k), _rows_ok(v)
        if ext_idx is not None:
            k_ext, v_ext = _rows_ok(k_ext), _rows_ok(v_ext)
        tc_fwd = FWD_IMPL == "tc" and q.shape[2] == 128
        tc_bwd = BWD_IMPL == "tc" and q.shape[2] == 128
        # block-structured extras run as one more key tile on the tensor cores; both directions must take
        # that route (or neither), since the forward's statistics feed the backward either way
        block = int(ext_block) if (ext_idx is not None and tc_fwd and tc_bwd and BLOCK_EXTRAS and ext_block and 128 % int(ext_block) == 0
                                   and k_ext.shape[0] >= q.shape[0]) else 0
        if tc_fwd:
            from speculators_b200.ops import gemm_status

            out, lse2 = _ext.lib().attn_fwd_tc(q, k, v, lo, hi, k_ext, v_ext, ext_idx, scale, gemm_status(q.device), block, bool(ext_causal))
        else:
            out, lse2 = _ext.lib().attn_fwd(q, k, v, lo, hi, k_ext, v_ext, ext_idx, scale)
        ctx.save_for_backward(q, k, v, out, lse2, lo, hi, k_ext, v_ext, ext_idx)
        ctx.scale = scale
        ctx.block = (block, bool(ext_causal))
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse2, lo, hi, k_ext, v_ext, ext_idx = ctx.saved_tensors
        if BWD_IMPL == "tc" and q.shape[2] == 128:
            from speculators_b200.ops import gemm_status

            impl, status = 1, gemm_status(q.device)
        else:
            impl, status = 0, None
        dq, dk, dv, dke, dve = _ext.lib().attn_bwd(
            _rows_ok(dout), q, k, v, out, lse2, lo, hi, k_ext, v_ext, ext_idx, ctx.scale, impl, status, ctx.block[0], ctx.block[1])
        if ext_idx is not None:
            return dq, dk, dv, None, None, dke.to(q.dtype), dve.to(q.dtype), None, None, None, None
        return dq, dk, dv, None, None, None, None, None, None, None, None


def masked_attention_cuda(q, k_ctx, v_ctx, spec: AttnSpec, k_ext=None, v_ext=None, scale=None):
    hd = q.shape[-1]
    scale = hd**-0.5 if scale is None else float(scale)
    if hd not in _SUPPORTED_HEAD_DIMS or q.dtype != torch.bfloat16:
        return masked_attention_reference(q, k_ctx, v_ctx, spec, k_ext, v_ext, scale)
    ext_idx = spec.extra_idx
    if ext_idx is None or k_ext is None or ext_idx.shape[1] == 0:
        ext_idx = k_ext = v_ext = None
    else:
        ext_idx = ext_idx.to(torch.int32).contiguous()
    block = getattr(spec, "extra_block", 0) if ext_idx is not None else 0
    return _MaskedAttentionFn.apply(q, k_ctx, v_ctx, spec.lo, spec.hi, k_ext, v_ext, ext_idx, scale, block, bool(getattr(spec, "extra_block_causal", False)))
