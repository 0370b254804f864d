"""Algorithm implementations.  Importing this package registers every model and
config class with ``SpeculatorModel.registry`` / ``SpeculatorModelConfig.registry``
(explicit imports, like src/speculators/models/__init__.py:3-7)."""

from speculators_b200.models import eagle3  # noqa: F401

__all__ = ["eagle3"]
