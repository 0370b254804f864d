"""Conversion of external speculative-decoding checkpoints (EAGLE-3 research layout,
DFlash, verifier checkpoints with MTP heads) into this package's checkpoint format
(parity: src/speculators/convert/__init__.py)."""

from speculators_b200.convert.entrypoints import convert_model

__all__ = ["convert_model"]
