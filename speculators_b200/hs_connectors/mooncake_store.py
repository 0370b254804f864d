"""Module name under which the reference ships its integrity-checked Mooncake store
(hs_connectors/src/hs_connectors/mooncake_store.py); the implementation lives in ``store``."""

from speculators_b200.hs_connectors import store as _impl
from speculators_b200.hs_connectors.store import *  # noqa: F401,F403

__all__ = list(_impl.__all__)
