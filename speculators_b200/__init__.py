"""B200-native training framework for speculative-decoding draft models."""

from speculators_b200.config import SpeculatorModelConfig, SpeculatorsConfig, VerifierConfig, reload_schemas
from speculators_b200.model import SpeculatorModel
from speculators_b200.proposals import GreedyTokenProposalConfig, TokenProposalConfig
from speculators_b200.version import __version__

from speculators_b200 import models  # noqa: E402, F401  (registers the algorithms)
from speculators_b200.models.eagle3 import Eagle3DraftModel, Eagle3SpeculatorConfig  # noqa: E402

__all__ = [
    "Eagle3DraftModel",
    "Eagle3SpeculatorConfig",
    "GreedyTokenProposalConfig",
    "SpeculatorModel",
    "SpeculatorModelConfig",
    "SpeculatorsConfig",
    "TokenProposalConfig",
    "VerifierConfig",
    "__version__",
    "reload_schemas",
]
