"""Training losses: dense (``eager``), fused-kernel (``fused``) and the shared
selection / weighting / reduction helpers.

The package namespace re-exports the helpers of ``losses.utils`` grouped by role; the
per-position loss terms themselves are re-exported from there too, so
``from speculators_b200.losses import kl_div_loss`` keeps working whichever implementation
``resolve_loss_config`` picks.
"""

from speculators_b200.losses import utils as _utils

_TERMS = ("kl_div_loss", "reverse_kl_div_loss", "js_div_loss", "ce_loss", "tv_loss", "neg_log_acceptance_loss", "lk_hybrid_loss")
_POSITION_WEIGHTS = ("exp_loss_decay", "dflash_loss_decay", "dpace_loss_decay")
_SELECTION = ("LossConfig", "resolve_loss_config", "loss_name_of")
_REDUCTION = ("reduce_masked", "loss_function", "compound_loss")

__all__ = sorted(_TERMS + _POSITION_WEIGHTS + _SELECTION + _REDUCTION)
globals().update({name: getattr(_utils, name) for name in __all__})
