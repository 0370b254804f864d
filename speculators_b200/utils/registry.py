"""Name -> class registries.

Every pluggable family in the framework (speculator models, speculator configs,
token-proposal configs, hidden-state backends) keeps one registry on its base
class.  A subclass of the base owns its *own* table, so registering an EAGLE-3
model never shows up in the proposal-config table.

Behavioural parity with the reference's ``ClassRegistryMixin``
(src/speculators/utils/registry.py:78-186): ``register(name)`` decorator,
``register_decorator`` bare decorator, duplicate names rejected,
``registered_classes()`` raising before anything is registered.  The storage
differs: each base gets its table lazily through ``__init_subclass__`` lookups
instead of a shared class attribute that is rebound on first use.
"""

from __future__ import annotations

from typing import Any, Callable, ClassVar

__all__ = ["ClassRegistryMixin"]


class ClassRegistryMixin:
    registry: ClassVar[dict[str, type[Any]] | None] = None
    registry_auto_discovery: ClassVar[bool] = False
    registry_populated: ClassVar[bool] = False

    @classmethod
    def _table(cls, create: bool) -> dict[str, type[Any]] | None:
        table = cls.registry
        if table is None and create:
            table = {}
            cls.registry = table
        return table

    @classmethod
    def register(cls, name: str | None = None) -> Callable[[type[Any]], type[Any]]:
        if name is not None and not isinstance(name, str):
            raise ValueError(f"register: name must be a string or None; got name={name!r}")

        def _apply(klass: type[Any]) -> type[Any]:
            return cls.register_decorator(klass, name=name)

        return _apply

    @classmethod
    def register_decorator(cls, clazz: type[Any], name: str | None = None) -> type[Any]:
        if not isinstance(clazz, type):
            raise TypeError(
                f"register_decorator must be used as a class decorator; got {clazz!r}. "
                "Use @Base.register('name') or @Base.register_decorator."
            )
        if name is not None and not isinstance(name, str):
            raise ValueError(f"register_decorator must be used as a class decorator with a name that is a string or None; got name={name!r}")
        key = name or clazz.__name__
        table = cls._table(create=True)
        assert table is not None
        if key in table:
            raise ValueError(
                f"{key!r} is already registered in the {cls.__name__} registry as {table[key]!r}; "
                f"refusing to replace it with {clazz!r}"
            )
        table[key] = clazz
        return clazz

    @classmethod
    def registered_classes(cls) -> tuple[type[Any], ...]:
        table = cls._table(create=False)
        if table is None:
            raise ValueError(
                f"{cls.__name__}.registered_classes() must be called after registering classes "
                "(nothing is registered yet)"
            )
        return tuple(table.values())

    @classmethod
    def registered_name(cls, clazz: type[Any]) -> str | None:
        """Reverse lookup: the name ``clazz`` was registered under, if any."""
        for key, value in (cls._table(create=False) or {}).items():
            if value is clazz:
                return key
        return None
