"""Noise augmentation of the verifier hidden states, applied to the training split only
(src/speculators/train/noise_transforms.py).

A transform is a callable on the sample dict.  It perturbs the tensors named in ``tensors``
(by default the draft's input hidden states) with zero-mean noise of scale ``std`` and leaves
every other entry alone; the noise is drawn in the tensor's own dtype and device, so the
transform works in data-loader workers and on device tensors alike.
"""

from __future__ import annotations

from collections.abc import Iterable

import torch

__all__ = ["AddGaussianNoise", "AddUniformNoise", "TransformTensors"]


class TransformTensors:
    """Base: ``transform`` maps one tensor; ``__call__`` applies it to the selected entries."""

    def __init__(self, std: float = 0.05, tensors: Iterable[str] = ("hidden_states",)):
        self.std = float(std)
        self.tensors = tuple(tensors)

    def transform(self, tensor: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("Subclasses must implement this method")

    def __call__(self, data: dict) -> dict:
        data.update({name: self.transform(data[name]) for name in self.tensors})
        return data

    def __repr__(self) -> str:
        return f"{type(self).__name__}(std={self.std}, tensors={self.tensors})"


class AddUniformNoise(TransformTensors):
    """``x + u``, ``u`` uniform in ``[-std, std]`` (the trainer's default, ``--noise-std``)."""

    def transform(self, tensor: torch.Tensor) -> torch.Tensor:
        noise = torch.empty_like(tensor).uniform_(-self.std, self.std) if self.std > 0 else torch.zeros_like(tensor)
        return tensor + noise


class AddGaussianNoise(TransformTensors):
    """``x + std * n``, ``n`` standard normal."""

    def transform(self, tensor: torch.Tensor) -> torch.Tensor:
        return torch.add(tensor, torch.randn_like(tensor), alpha=self.std)
