"""Masked attention with a per-row mask description.

Every attention pattern of the supported algorithms decomposes, per query row
``i``, into

* a contiguous window ``[lo[i], hi[i])`` of *context* keys (causal, same-document
  and sliding-window constraints all intersect to an interval), plus
* a short list of individually addressed *extra* keys ``extra_idx[i, :]``
  (``-1`` = unused slot): the per-step diagonal keys of EAGLE-3's
  training-time-test, the same-rollout keys of P-EAGLE, the in-block noise keys
  of DFlash / DSpark.

``AttnSpec`` carries those three arrays.  This replaces the reference's
``mask_mod`` closures + ``BlockMask`` (src/speculators/models/eagle3/attention.py:
11-112, peagle/attention.py:46-72, dflash/attention.py:7-100): the spec is built
by small fixed-shape device ops from ``document_ids`` / anchors, needs no
host sync and no compiled mask builder, and the kernel derives its KV tile range
per query tile from ``lo`` / ``hi`` directly.

``masked_attention_reference`` is the dense fp32 formulation (differentiable
through autograd); it is the oracle for the CUDA kernels and the CPU path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

__all__ = ["AttnSpec", "masked_attention", "masked_attention_reference"]


@dataclass
class AttnSpec:
    lo: torch.Tensor  # int32 [Tq]   first allowed context key
    hi: torch.Tensor  # int32 [Tq]   one past the last allowed context key
    extra_idx: torch.Tensor | None = None  # int32 [Tq, E] rows of the extra K/V, -1 = none
    # When the extra keys have block structure - row r lists exactly the rows of its own block of `extra_block` rows
    # of the extra K/V (with `extra_block_causal`: only those up to r) - the builder says so here: the tcgen05
    # kernels then run a query tile's extras as one block-diagonal key tile on the tensor cores instead of
    # gathering them row by row.  `extra_idx` stays authoritative for every other path.
    extra_block: int = 0
    extra_block_causal: bool = False

    def dense(self, n_ctx: int, n_extra: int = 0) -> torch.Tensor:
        """Boolean [Tq, n_ctx + n_extra] mask equivalent to this spec (tests/oracle)."""
        j = torch.arange(n_ctx, device=self.lo.device)
        m = (j[None, :] >= self.lo[:, None]) & (j[None, :] < self.hi[:, None])
        if n_extra:
            e = torch.zeros(self.lo.shape[0], n_extra, dtype=torch.bool, device=self.lo.device)
            if self.extra_idx is not None:
                idx = self.extra_idx.long()
                valid = idx >= 0
                rows = torch.arange(idx.shape[0], device=idx.device)[:, None].expand_as(idx)
                e[rows[valid], idx[valid]] = True
            m = torch.cat([m, e], dim=1)
        return m


def masked_attention_reference(q, k_ctx, v_ctx, spec: AttnSpec, k_ext=None, v_ext=None, scale=None):
    """q [Tq, nh, hd]; k/v_ctx [Tc, nkv, hd]; k/v_ext [Te, nkv, hd] -> [Tq, nh, hd].

    Softmax in fp32 over the allowed context interval and the listed extra keys.
    A row with no allowed key returns zeros.
    """
    Tq, nh, hd = q.shape
    nkv = k_ctx.shape[1]
    rep = nh // nkv
    scale = hd**-0.5 if scale is None else scale
    qf = q.float().transpose(0, 1)  # [nh, Tq, hd]
    kf = k_ctx.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    vf = v_ctx.float().transpose(0, 1).repeat_interleave(rep, dim=0)
    s_ctx = torch.matmul(qf, kf.transpose(1, 2)) * scale  # [nh, Tq, Tc]
    Tc = k_ctx.shape[0]
    j = torch.arange(Tc, device=q.device)
    allow = (j[None, :] >= spec.lo[:, None]) & (j[None, :] < spec.hi[:, None])
    s_ctx = s_ctx.masked_fill(~allow[None], float("-inf"))
    have_ext = spec.extra_idx is not None and k_ext is not None and spec.extra_idx.shape[1] > 0
    if have_ext:
        idx = spec.extra_idx.long()
        valid = idx >= 0
        safe = idx.clamp(min=0)
        ke = k_ext.float()[safe].repeat_interleave(rep, dim=2)  # [Tq, E, nh, hd]
        ve = v_ext.float()[safe].repeat_interleave(rep, dim=2)
        s_ext = torch.einsum("hqd,qehd->hqe", qf, ke) * scale
        s_ext = s_ext.masked_fill(~valid[None], float("-inf"))
        s_all = torch.cat([s_ctx, s_ext], dim=-1)
    else:
        s_all = s_ctx
    row_max = s_all.amax(dim=-1, keepdim=True)
    row_max = torch.where(torch.isfinite(row_max), row_max, torch.zeros_like(row_max))
    p = torch.exp(s_all - row_max)
    denom = p.sum(-1, keepdim=True)
    p = p / torch.where(denom > 0, denom, torch.ones_like(denom))
    out = torch.matmul(p[..., :Tc], vf)
    if have_ext:
        out = out + torch.einsum("hqe,qehd->hqd", p[..., Tc:], ve)
    return out.transpose(0, 1).to(q.dtype)


def masked_attention(q, k_ctx, v_ctx, spec: AttnSpec, k_ext=None, v_ext=None, scale=None):
    """Dispatch: CUDA tensors run the sm_100a kernel, CPU tensors the dense oracle."""
    if q.is_cuda:
        from speculators_b200.ops import attention_cuda

        return attention_cuda.masked_attention_cuda(q, k_ctx, v_ctx, spec, k_ext, v_ext, scale)
    return masked_attention_reference(q, k_ctx, v_ctx, spec, k_ext, v_ext, scale)
