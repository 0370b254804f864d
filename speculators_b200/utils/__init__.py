from speculators_b200.utils.pydantic_utils import (
    PydanticClassRegistryMixin,
    ReloadableBaseModel,
)
from speculators_b200.utils.registry import ClassRegistryMixin

__all__ = ["ClassRegistryMixin", "PydanticClassRegistryMixin", "ReloadableBaseModel"]
