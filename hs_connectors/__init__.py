"""``hs_connectors``: the import name of the reference's stand-alone hidden-state transport
package (its top-level ``hs_connectors/`` project).  Here the transports are part of
``speculators_b200``; this package maps the old import paths onto them, so a vLLM launch
configuration or a script written against ``hs_connectors.*`` keeps working:

    from hs_connectors import HiddenStatesBackend, FileTransfer
    kv_connector_module_path = "hs_connectors.mooncake_hidden_states_connector"
"""

import importlib
import sys

from speculators_b200.hs_connectors import *  # noqa: F401,F403
from speculators_b200.hs_connectors import __all__ as _exported
from speculators_b200.version import __version__  # noqa: F401

__all__ = list(_exported)

for _name in ("transfer", "mooncake_store", "mooncake_hidden_states_connector", "store", "mooncake", "nvlink", "vllm_connector"):
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"speculators_b200.hs_connectors.{_name}")
    globals()[_name] = sys.modules[f"{__name__}.{_name}"]
