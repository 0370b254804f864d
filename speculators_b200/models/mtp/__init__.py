from speculators_b200.models.mtp.config import MTPSpeculatorConfig
from speculators_b200.models.mtp.core import MTPDraftModel, compute_step_weights
from speculators_b200.models.mtp.data import shift_batch_mtp

__all__ = ["MTPDraftModel", "MTPSpeculatorConfig", "compute_step_weights", "shift_batch_mtp"]
