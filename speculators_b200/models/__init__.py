"""Algorithm implementations.  Importing this package registers every model and
config class with ``SpeculatorModel.registry`` / ``SpeculatorModelConfig.registry``
(explicit imports, like src/speculators/models/__init__.py:3-7)."""

from speculators_b200.models import dflash, dspark, eagle3, mtp, peagle  # noqa: F401
from speculators_b200.models.dflash import DFlashDraftModel, DFlashSpeculatorConfig
from speculators_b200.models.dspark import DSparkDraftModel, DSparkSpeculatorConfig
from speculators_b200.models.eagle3 import Eagle3DraftModel, Eagle3SpeculatorConfig
from speculators_b200.models.mtp import MTPDraftModel, MTPSpeculatorConfig
from speculators_b200.models.peagle import PEagleDraftModel, PEagleSpeculatorConfig

__all__ = [
    "DFlashDraftModel", "DFlashSpeculatorConfig", "DSparkDraftModel", "DSparkSpeculatorConfig", "Eagle3DraftModel",
    "Eagle3SpeculatorConfig", "MTPDraftModel", "MTPSpeculatorConfig", "PEagleDraftModel", "PEagleSpeculatorConfig",
    "dflash", "dspark", "eagle3", "mtp", "peagle",
]
