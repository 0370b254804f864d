from speculators_b200.models.dflash.config import DFlashSpeculatorConfig
from speculators_b200.models.dflash.core import DFlashDraftModel

__all__ = ["DFlashDraftModel", "DFlashSpeculatorConfig"]
