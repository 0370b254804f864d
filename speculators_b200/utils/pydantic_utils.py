"""Polymorphic pydantic models keyed by a discriminator field.

``Base.model_validate({"kind": "x", ...})`` returns an instance of the subclass
registered as ``"x"``.  The reference gets this by rebuilding a tagged-union core
schema every time the registry changes (src/speculators/utils/pydantic_utils.py:
41-194, ``reload_schema``).  Here the dispatch happens at validation time in a
``wrap`` validator on the base class, so a subclass registered after import is
picked up without any schema rebuild; ``reload_schema`` is kept as a cheap
``model_rebuild`` for API parity.  In the other direction a ``wrap`` serializer makes a
field declared with the family's base type dump the fields of the concrete subclass it
holds (pydantic alone would serialize by the declared type and drop them).
"""

from __future__ import annotations

import threading
from typing import Any, ClassVar

from pydantic import BaseModel, model_serializer, model_validator

from speculators_b200.utils.registry import ClassRegistryMixin

__all__ = ["PydanticClassRegistryMixin", "ReloadableBaseModel"]


class ReloadableBaseModel(BaseModel):
    @classmethod
    def reload_schema(cls) -> None:
        cls.model_rebuild(force=True)


class PydanticClassRegistryMixin(ReloadableBaseModel, ClassRegistryMixin):
    schema_discriminator: ClassVar[str] = "model_type"
    # Base(tag=...) builds the registered subclass; families whose base must stay constructible
    # as itself switch this off
    dispatch_on_construct: ClassVar[bool] = True

    @classmethod
    def __pydantic_schema_base_type__(cls) -> type[Any]:
        """Root of the polymorphic family: the first class in the MRO (walking up
        from ``cls``) that declares ``schema_discriminator`` in its own body."""
        root = cls
        for klass in cls.__mro__:
            if "schema_discriminator" in vars(klass) and klass is not PydanticClassRegistryMixin:
                root = klass
        return root

    def __new__(cls, *args: Any, **kwargs: Any):
        """Constructing the family's base class with the tag of a registered subclass builds
        that subclass: ``Base(kind="x", ...)`` is ``X(kind="x", ...)``."""
        target = cls
        if kwargs and cls.dispatch_on_construct and cls is cls.__pydantic_schema_base_type__():
            tag = kwargs.get(cls.schema_discriminator)
            found = (cls.registry or {}).get(tag) if isinstance(tag, str) else None
            if found is not None and issubclass(found, cls):
                target = found
        return super().__new__(target)

    def __init__(self, **data: Any) -> None:
        # tell the validator below that this object already has its final class (``__new__`` chose
        # it): it must fill *this* instance instead of building another one
        _CONSTRUCTION.stack.append(True)
        try:
            super().__init__(**data)
        finally:
            _CONSTRUCTION.stack.pop()

    @classmethod
    def register_decorator(cls, clazz: type[Any], name: str | None = None) -> type[Any]:
        if not (isinstance(clazz, type) and issubclass(clazz, BaseModel)):
            raise TypeError(f"{clazz!r} is not a subclass of Pydantic BaseModel")
        return super().register_decorator(clazz, name=name)

    @model_validator(mode="wrap")
    @classmethod
    def _dispatch_on_discriminator(cls, value: Any, handler):  # noqa: ANN001
        if isinstance(value, cls) or not isinstance(value, dict):
            return handler(value)
        if _CONSTRUCTION.stack and _CONSTRUCTION.stack[-1]:
            _CONSTRUCTION.stack[-1] = False  # only the object under construction; its nested fields dispatch normally
            return handler(value)
        root = cls.__pydantic_schema_base_type__()
        if cls is not root:
            return handler(value)  # already the concrete class
        table = root.registry or {}
        tag = value.get(root.schema_discriminator)
        target = table.get(tag) if isinstance(tag, str) else None
        if target is None or target is cls:
            if table and tag is not None and tag not in table and tag != "":
                raise ValueError(
                    f"unknown {root.schema_discriminator}={tag!r}; registered: "
                    f"{sorted(table)}"
                )
            return handler(value)
        return target.model_validate(value)

    @model_serializer(mode="wrap")
    def _serialize_as_own_class(self, handler, info):  # noqa: ANN001
        data = handler(self)
        own = type(self)
        if not isinstance(data, dict) or id(self) in _RESERIALIZING or info.include or info.exclude:
            return data
        if all(name in data for name in own.model_fields):
            return data
        # fields are missing: dropped by the caller's exclude_* flags, or because this instance
        # was reached through a field typed as a base class; dumping with the instance's own
        # schema and the same flags is right in both cases
        _RESERIALIZING.add(id(self))
        try:
            return own.__pydantic_serializer__.to_python(
                self, mode=info.mode, by_alias=info.by_alias, exclude_unset=info.exclude_unset, exclude_defaults=info.exclude_defaults,
                exclude_none=info.exclude_none, round_trip=info.round_trip, warnings=False)
        finally:
            _RESERIALIZING.discard(id(self))


_RESERIALIZING: set[int] = set()
class _ConstructionStack(threading.local):
    def __init__(self) -> None:
        self.stack: list[bool] = []


_CONSTRUCTION = _ConstructionStack()
