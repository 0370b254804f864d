from speculators_b200.models.mtp.config import MTPSpeculatorConfig
from speculators_b200.models.mtp.core import MTPDraftModel, compute_step_weights

__all__ = ["MTPDraftModel", "MTPSpeculatorConfig", "compute_step_weights"]
