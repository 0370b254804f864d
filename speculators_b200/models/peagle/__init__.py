from speculators_b200.models.peagle.config import PEagleSpeculatorConfig
from speculators_b200.models.peagle.core import PEagleDraftModel

__all__ = ["PEagleDraftModel", "PEagleSpeculatorConfig"]
