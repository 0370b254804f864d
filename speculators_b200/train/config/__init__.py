from speculators_b200.train.config.schema import TrainConfig

__all__ = ["TrainConfig"]
