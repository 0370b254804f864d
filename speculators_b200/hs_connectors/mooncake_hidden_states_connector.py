"""Module name under which the reference ships its vLLM connector
(hs_connectors/mooncake_hidden_states_connector.py); launch configurations that name it as
``kv_connector_module_path`` keep working.  The implementation lives in ``vllm_connector``."""

from speculators_b200.hs_connectors import vllm_connector as _impl
from speculators_b200.hs_connectors.vllm_connector import *  # noqa: F401,F403

__all__ = list(_impl.__all__)
