"""Algorithm implementations.  Importing this package registers every model and
config class with ``SpeculatorModel.registry`` / ``SpeculatorModelConfig.registry``
(explicit imports, like src/speculators/models/__init__.py:3-7)."""

from speculators_b200.models import dflash, dspark, eagle3, mtp, peagle  # noqa: F401

__all__ = ["dflash", "dspark", "eagle3", "mtp", "peagle"]
