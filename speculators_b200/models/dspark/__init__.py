from speculators_b200.models.dspark.config import DSparkSpeculatorConfig
from speculators_b200.models.dspark.core import DSparkDraftModel

__all__ = ["DSparkDraftModel", "DSparkSpeculatorConfig"]
