"""Pluggable transports for verifier -> trainer hidden states."""

from speculators_b200.hs_connectors.mooncake import MooncakeBackend, MooncakeTransfer
from speculators_b200.hs_connectors.nvlink import HiddenStateRing, HiddenStateRingWriter, NvlinkBackend, NvlinkTransfer
from speculators_b200.hs_connectors.store import (
    DictStoreClient, HiddenStatesStore, MooncakeHiddenStatesStore, MooncakeIntegrityError, MooncakeStoreConfig,
    NonFiniteTensorError, assert_finite,
)
from speculators_b200.hs_connectors.transfer import (
    FileBackend, FileTransfer, HiddenStatesBackend, HiddenStatesTransfer, wait_for_lock,
)

__all__ = [
    "DictStoreClient", "FileBackend", "FileTransfer", "HiddenStateRing", "HiddenStateRingWriter", "HiddenStatesBackend", "NvlinkBackend",
    "NvlinkTransfer", "HiddenStatesStore", "HiddenStatesTransfer",
    "MooncakeBackend", "MooncakeHiddenStatesStore", "MooncakeIntegrityError", "MooncakeStoreConfig", "MooncakeTransfer",
    "NonFiniteTensorError", "assert_finite", "wait_for_lock",
]
