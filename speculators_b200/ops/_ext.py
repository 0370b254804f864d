"""Loading of the native extension.

``lib()`` returns ``torch.ops.sb200`` after making sure ``_sb200.so`` (or, with
``SB200_CHECKED_BUILD=1``, the index-checking debug flavour ``_sb200_checked.so``) is loaded.
On a machine with a GPU the extension is mandatory: if the shared object is
missing or stale it is rebuilt in-tree, and a failure to do so raises instead
of silently running the PyTorch reference path.
"""

from __future__ import annotations

import threading

import torch

from speculators_b200.ops import _build

_lock = threading.Lock()
_loaded = False


def available() -> bool:
    return _loaded or _build.active_lib().exists()


def lib():
    global _loaded
    if not _loaded:
        with _lock:
            if not _loaded:
                if not _build.is_current():
                    _build.build()
                torch.ops.load_library(str(_build.active_lib()))
                _loaded = True
    return torch.ops.sb200


def loaded_library_path() -> str | None:
    return str(_build.active_lib()) if _loaded else None
