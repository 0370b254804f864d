"""Learning-rate schedules as pure functions of the step index.

``linear`` and ``cosine`` reproduce the multipliers of Hugging Face's
``get_linear_schedule_with_warmup`` / ``get_cosine_schedule_with_warmup`` that the
reference uses (src/speculators/train/trainer.py:338-376); warm-up / total step
resolution follows ``_resolve_scheduler_steps`` (:128-163).  The engine takes the
learning rate as a per-step value, so a schedule has no optimizer to wrap and its
whole state is the step counter.
"""

from __future__ import annotations

import math
import warnings

__all__ = ["LRSchedule", "resolve_scheduler_steps"]


def resolve_scheduler_steps(config, train_loader_len: int) -> tuple[int, int]:
    total = config.scheduler_total_steps if config.scheduler_total_steps is not None else config.num_epochs * train_loader_len
    if config.scheduler_warmup_steps is not None:
        if config.scheduler_warmup_ratio is not None:
            warnings.warn("Both scheduler_warmup_steps and scheduler_warmup_ratio are set; using scheduler_warmup_steps.", stacklevel=2)
        return config.scheduler_warmup_steps, total
    if config.scheduler_warmup_ratio is not None:
        if not 0 <= config.scheduler_warmup_ratio <= 1:
            raise ValueError("scheduler_warmup_ratio must be between 0 and 1.")
        return int(total * config.scheduler_warmup_ratio), total
    return total // 100, total


class LRSchedule:
    def __init__(self, kind: str, base_lr: float, warmup_steps: int = 0, total_steps: int = 1, num_cycles: float = 0.5):
        if kind not in ("linear", "cosine", "none"):
            raise ValueError(f"unknown scheduler_type {kind!r}")
        self.kind, self.base_lr = kind, base_lr
        self.warmup_steps, self.total_steps, self.num_cycles = warmup_steps, total_steps, num_cycles
        self.last_step = 0

    def multiplier(self, step: int) -> float:
        if self.kind == "none":
            return 1.0
        if step < self.warmup_steps:
            return step / max(1, self.warmup_steps)
        span = max(1, self.total_steps - self.warmup_steps)
        if self.kind == "linear":
            return max(0.0, (self.total_steps - step) / span)
        progress = (step - self.warmup_steps) / span
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * self.num_cycles * 2.0 * progress)))

    def current_lr(self) -> float:
        return self.base_lr * self.multiplier(self.last_step)

    def step(self) -> None:
        self.last_step += 1

    def state_dict(self) -> dict:
        return {"last_step": self.last_step, "kind": self.kind, "base_lr": self.base_lr,
                "warmup_steps": self.warmup_steps, "total_steps": self.total_steps, "num_cycles": self.num_cycles}

    def load_state_dict(self, sd: dict) -> None:
        self.last_step = int(sd.get("last_step", sd.get("last_epoch", 0)))
