"""Batch adapter for MTP: the head consumes the verifier's *last* hidden states
under the name ``hidden_states`` and needs no positional shift
(src/speculators/models/mtp/data.py)."""

__all__ = ["shift_batch_mtp"]


def shift_batch_mtp(batch: dict) -> dict:
    out = dict(batch)
    if "verifier_last_hidden_states" in out:
        out["hidden_states"] = out.pop("verifier_last_hidden_states")
    return out
