from speculators_b200.models.eagle3.config import Eagle3SpeculatorConfig
from speculators_b200.models.eagle3.core import Eagle3DraftModel, Eagle3FirstLayer
from speculators_b200.models.eagle3.data import shift_batch

__all__ = ["Eagle3DraftModel", "Eagle3FirstLayer", "Eagle3SpeculatorConfig", "shift_batch"]
