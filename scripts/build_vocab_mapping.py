#!/usr/bin/env python3
"""Build the draft<->target vocabulary maps from a token-frequency table.

Writes ``d2t.npy`` (per draft id: offset to its target id) and ``t2d.npy`` (per target
id: is it in the draft vocabulary) — the files ``scripts/train.py`` looks for.

    python scripts/build_vocab_mapping.py --token-freq-path ./output/token_freq.pt \\
        --draft-vocab-size 32000 --target-vocab-size 128256 --output-path ./output

CLI parity: scripts/build_vocab_mapping.py:35 of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import logging
import sys
from pathlib import Path

import numpy as np
import torch

from speculators_b200.train.vocab_mapping import build_vocab_mappings_from_distribution, get_target_vocab_size

logger = logging.getLogger(__name__)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Build vocabulary mappings from a token frequency distribution")
    ap.add_argument("--token-freq-path", default="./output/token_freq.pt")
    ap.add_argument("--draft-vocab-size", type=int, required=True)
    ap.add_argument("--target-vocab-size", type=int, default=None)
    ap.add_argument("--target-model-path", default=None, help="read the target vocabulary size from this model's config")
    ap.add_argument("--output-path", default="./output")
    return ap


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    """Parsed command line (``sys.argv`` when ``argv`` is None)."""
    return build_parser().parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s - %(name)s - %(levelname)s - %(message)s")
    args = build_parser().parse_args(argv)
    src = Path(args.token_freq_path)
    if not src.exists():
        raise FileNotFoundError(f"Token frequency file not found: {src}")
    freq = torch.load(src, weights_only=True)
    d2t, t2d = build_vocab_mappings_from_distribution(
        token_freq_dict=freq, draft_vocab_size=args.draft_vocab_size,
        target_vocab_size=get_target_vocab_size(args.target_vocab_size, args.target_model_path),
    )
    dst = Path(args.output_path)
    dst.mkdir(parents=True, exist_ok=True)
    for name, tensor in (("d2t", d2t), ("t2d", t2d)):
        np.save(dst / f"{name}.npy", tensor.cpu().numpy())
        logger.info("Saved %s to %s (shape: %s)", name, dst / f"{name}.npy", tuple(tensor.shape))
    return 0


if __name__ == "__main__":
    sys.exit(main())
