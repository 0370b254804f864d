from speculators_b200.models.eagle3.config import Eagle3SpeculatorConfig
from speculators_b200.models.eagle3.core import Eagle3DraftModel, Eagle3FirstLayer

__all__ = ["Eagle3DraftModel", "Eagle3FirstLayer", "Eagle3SpeculatorConfig"]
