from speculators_b200.parallel.distributed import (
    get_dp_group, get_dp_rank, get_dp_size, get_local_rank, get_rank, get_sp_group, get_sp_rank,
    get_sp_size, get_world_size, is_distributed, maybe_destroy_distributed, maybe_setup_distributed,
)
from speculators_b200.parallel.engine import EngineConfig, TrainEngine, split_named_params_for_muon

__all__ = [
    "EngineConfig", "TrainEngine", "get_dp_group", "get_dp_rank", "get_dp_size", "get_local_rank",
    "get_rank", "get_sp_group", "get_sp_rank", "get_sp_size", "get_world_size", "is_distributed",
    "maybe_destroy_distributed", "maybe_setup_distributed", "split_named_params_for_muon",
]
