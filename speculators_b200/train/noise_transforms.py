"""Noise augmentation of the verifier hidden states (training split only)
(src/speculators/train/noise_transforms.py)."""

import torch

__all__ = ["AddGaussianNoise", "AddUniformNoise", "TransformTensors"]


class TransformTensors:
    def __init__(self, std: float = 0.05, tensors=("hidden_states",)):
        self.std, self.tensors = std, tuple(tensors)

    def __call__(self, data: dict) -> dict:
        for name in self.tensors:
            data[name] = self.transform(data[name])
        return data

    def transform(self, tensor: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("Subclasses must implement this method")


class AddGaussianNoise(TransformTensors):
    def transform(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor + torch.randn_like(tensor) * self.std


class AddUniformNoise(TransformTensors):
    """Uniform in ``[-std, std]``."""

    def transform(self, tensor: torch.Tensor) -> torch.Tensor:
        return tensor + (torch.rand_like(tensor) * 2.0 - 1.0) * self.std
