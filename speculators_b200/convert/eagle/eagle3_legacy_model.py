"""``Eagle3Speculator``: the name converted EAGLE-3 checkpoints carry in their
``architectures`` field, with the constructor of the reference's conversion-time model
(src/speculators/convert/eagle/eagle3_legacy_model.py: ``verifier``,
``verifier_attachment_mode``, ``reduce_vocab_size``, ``has_drafter_embedding``).  Here it
is the training model itself (``Eagle3DraftModel``) under that signature, so a checkpoint
written by the converter loads, runs and re-saves through one implementation; the
reference keeps a separate, deprecated single-step module for this."""

from __future__ import annotations

import os
from typing import Any

from speculators_b200.models.eagle3 import Eagle3DraftModel, Eagle3SpeculatorConfig

__all__ = ["Eagle3Speculator"]


class Eagle3Speculator(Eagle3DraftModel):
    def __init__(self, config: Eagle3SpeculatorConfig, verifier: str | os.PathLike | None = None,
                 verifier_attachment_mode: str | None = None, reduce_vocab_size: bool = True, has_drafter_embedding: bool = True):
        """``verifier`` / ``verifier_attachment_mode``: accepted for signature parity; the draft
        never holds the verifier (``"detached"`` is the only mode), its name lives in
        ``config.speculators_config.verifier``.  ``reduce_vocab_size=False`` drops the
        draft-to-target vocabulary maps (draft and target vocabularies coincide);
        ``has_drafter_embedding=False`` marks the embedding as taken from the verifier
        (it is then not trained)."""
        if verifier_attachment_mode not in (None, "detached"):
            raise ValueError(f"verifier_attachment_mode={verifier_attachment_mode!r} is not supported: the draft model is always detached")
        super().__init__(config)
        self.reduce_vocab_size, self.has_drafter_embedding = bool(reduce_vocab_size), bool(has_drafter_embedding)
        if not has_drafter_embedding:
            self.embed_tokens.weight.requires_grad_(False)
        if not reduce_vocab_size:
            for name in ("d2t", "t2d"):
                if name in self._buffers:
                    self._buffers[name] = None

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, *args: Any, verifier: str | None = None,
                        verifier_attachment_mode: str | None = None, **kwargs: Any):
        if verifier_attachment_mode not in (None, "detached"):
            raise ValueError(f"verifier_attachment_mode={verifier_attachment_mode!r} is not supported: the draft model is always detached")
        return Eagle3DraftModel.from_pretrained(pretrained_model_name_or_path, *args, verifier=verifier, **kwargs)
