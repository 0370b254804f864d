"""Training runtime: trainer, checkpointing, schedules, data pipeline, config."""

from speculators_b200.train.checkpointer import Checkpointer, DistributedCheckpointer, SingleGPUCheckpointer
from speculators_b200.train.trainer import Trainer, TrainerConfig

__all__ = ["Checkpointer", "DistributedCheckpointer", "SingleGPUCheckpointer", "Trainer", "TrainerConfig"]
