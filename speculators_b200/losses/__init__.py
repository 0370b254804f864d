"""Training losses: dense (``eager``), fused-kernel (``fused``) and the shared
selection / weighting / reduction helpers."""

from speculators_b200.losses.utils import (
    LossConfig,
    ce_loss,
    compound_loss,
    dflash_loss_decay,
    dpace_loss_decay,
    exp_loss_decay,
    js_div_loss,
    kl_div_loss,
    lk_hybrid_loss,
    loss_function,
    loss_name_of,
    neg_log_acceptance_loss,
    reduce_masked,
    resolve_loss_config,
    reverse_kl_div_loss,
    tv_loss,
)

__all__ = [
    "LossConfig",
    "ce_loss",
    "compound_loss",
    "dflash_loss_decay",
    "dpace_loss_decay",
    "exp_loss_decay",
    "js_div_loss",
    "kl_div_loss",
    "lk_hybrid_loss",
    "loss_function",
    "loss_name_of",
    "neg_log_acceptance_loss",
    "reduce_masked",
    "resolve_loss_config",
    "reverse_kl_div_loss",
    "tv_loss",
]
