"""Loss selection, position weighting and masked reduction.

Parity targets (src/speculators/losses/utils.py): ``dflash_loss_decay`` :17-48,
``exp_loss_decay`` :51-61, ``dpace_loss_decay`` :64-112, ``resolve_loss_config``
:184-230 (a bare name or a JSON dict ``{"ce": 0.1, "tv": 0.9}``),
``compound_loss`` :233-266 and ``loss_function`` :269-304 (mask, decay,
``/ (mask.sum + 1e-5)``, batch mean).
"""

from __future__ import annotations

import json
from collections.abc import Callable

import torch

from speculators_b200.losses import eager, fused

_REDUCTION_EPS = 1e-5

LossFn = Callable[[torch.Tensor, torch.Tensor], torch.Tensor]
LossConfig = dict[str, tuple[LossFn, float]]


# ---- position weights -----------------------------------------------------------
def dflash_loss_decay(pos_idx: torch.Tensor, gamma: float, sample_from_anchor: bool = False, **_):
    """Block-position weights.  DFlash (slot 0 is the anchor itself): 0, 1,
    e^(-1/g), e^(-2/g), ...  DSpark (``sample_from_anchor``; slot 0 already predicts):
    1, e^(-1/g), e^(-2/g), ..."""
    pos = pos_idx.to(torch.float32) if not pos_idx.is_floating_point() else pos_idx
    if sample_from_anchor:
        return torch.exp(-pos / gamma)
    w = torch.exp(-(pos - 1).clamp(min=0) / gamma)
    return w * (pos != 0).to(w.dtype)


def exp_loss_decay(pos_idx: torch.Tensor, gamma: float, **_):
    return gamma**pos_idx


def dpace_loss_decay(pos_idx, loss_mask, block_size: int, dpace_alpha: float, elementwise_loss, **_):
    """D-PACE weights from per-position CE: confidence ``q = exp(-ce)`` smoothed to
    ``(1-a)q + a``, prefix product inside each block, then the suffix sum of the
    masked prefixes; masked slots weigh 0 and do not shrink the prefix."""
    del pos_idx
    with torch.no_grad():
        q = torch.exp(-elementwise_loss).float()
        if q.shape[1] % block_size:
            raise ValueError(f"sequence length {q.shape[1]} is not a multiple of block_size {block_size}")
        blocks = q.shape[1] // block_size
        q = q.reshape(blocks, block_size)
        mask = loss_mask.reshape(blocks, block_size).to(q.dtype)
        conf = torch.where(mask > 0, (1.0 - dpace_alpha) * q + dpace_alpha, torch.ones_like(q))
        prefix = torch.cumprod(conf, dim=-1) * mask
        suffix = prefix.flip(-1).cumsum(-1).flip(-1)
        return (suffix * mask).reshape(1, -1)


# ---- name -> function -------------------------------------------------------------
_FUSED: dict[str, LossFn] = {
    "kl_div": fused.fused_kl_div_loss,
    "rkl": fused.fused_reverse_kl_div_loss,
    "jsd": fused.fused_js_div_loss,
    "ce": fused.fused_ce_loss,
    "tv": fused.fused_tv_loss,
    "nla": fused.fused_nla_loss,
    "lk_hybrid": fused.fused_lk_hybrid_loss,
}
_EAGER: dict[str, LossFn] = {
    "kl_div": eager.kl_div_loss,
    "rkl": eager.reverse_kl_div_loss,
    "jsd": eager.js_div_loss,
    "ce": eager.ce_loss,
    "tv": eager.tv_loss,
    "nla": eager.neg_log_acceptance_loss,
    "lk_hybrid": eager.lk_hybrid_loss,
}
_IMPLS = {"fused": _FUSED, "eager": _EAGER}

kl_div_loss = fused.fused_kl_div_loss
reverse_kl_div_loss = fused.fused_reverse_kl_div_loss
js_div_loss = fused.fused_js_div_loss
ce_loss = fused.fused_ce_loss
tv_loss = fused.fused_tv_loss
neg_log_acceptance_loss = fused.fused_nla_loss
lk_hybrid_loss = fused.fused_lk_hybrid_loss


def loss_name_of(fn: LossFn) -> str | None:
    """Registered name of a loss function (either implementation), if any."""
    for table in _IMPLS.values():
        for name, cand in table.items():
            if cand is fn:
                return name
    return None


def resolve_loss_config(spec: str, implementation: str = "fused") -> LossConfig:
    table = _IMPLS.get(implementation)
    if table is None:
        raise ValueError(f"Unknown loss implementation '{implementation}'. Choose from: {sorted(_IMPLS)}")
    if spec in table:
        return {spec: (table[spec], 1.0)}
    try:
        parsed = json.loads(spec)
    except json.JSONDecodeError:
        raise ValueError(
            f"Unknown loss function '{spec}'. Pass a known name ({sorted(table)}) or a JSON dict "
            'of weights, e.g. \'{"ce": 0.1, "tv": 0.9}\'.'
        ) from None
    if not isinstance(parsed, dict) or not parsed:
        raise ValueError(f"Loss config must be a non-empty JSON dict of name -> weight. Got: {spec}")
    out: LossConfig = {}
    for name, weight in parsed.items():
        if name not in table:
            raise ValueError(f"Unknown loss function '{name}' in loss config. Choose from: {sorted(table)}")
        if isinstance(weight, bool) or not isinstance(weight, (int, float)):
            raise ValueError(f"Loss weight for '{name}' must be a number, got {type(weight).__name__}")
        out[name] = (table[name], float(weight))
    return out


# ---- reduction ------------------------------------------------------------------------
def reduce_masked(elementwise, loss_mask, pos_idx, decay_fn=None):
    mask = loss_mask.to(elementwise.dtype)
    weighted = elementwise * mask
    if decay_fn is not None:
        weighted = weighted * decay_fn(pos_idx.to(elementwise.dtype), elementwise_loss=weighted)
    return (weighted.sum(dim=1) / (mask.sum(dim=1) + _REDUCTION_EPS)).mean()


def loss_function(logits, targets, loss_mask, pos_idx, loss_fn: LossFn = kl_div_loss, decay_fn=None):
    return reduce_masked(loss_fn(logits, targets), loss_mask, pos_idx, decay_fn)


def compound_loss(logits, targets, loss_mask, pos_idx, loss_config: LossConfig, decay_fn=None):
    """Weighted sum of terms; per-term unweighted scalars are reported as
    ``"<name>_loss"`` only when there is more than one term."""
    total = torch.zeros((), device=logits.device, dtype=torch.float32)
    parts: dict[str, torch.Tensor] = {}
    for name, (fn, weight) in loss_config.items():
        term = loss_function(logits, targets, loss_mask, pos_idx, loss_fn=fn, decay_fn=decay_fn)
        if len(loss_config) > 1:
            parts[f"{name}_loss"] = term.detach()
        total = total + weight * term
    return total, parts
