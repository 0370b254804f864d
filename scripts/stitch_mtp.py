#!/usr/bin/env python3
"""Stitch fine-tuned MTP weights back into a verifier checkpoint.

    python scripts/stitch_mtp.py ./finetuned-mtp ./Qwen3-Next-80B-A3B-Instruct [--output-path ./out]

The verifier may be a local directory or a hub model id.  Output defaults to
``<verifier-name>-stitched`` in the current directory.  CLI parity:
scripts/stitch_mtp.py:303 of the reference.
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

from speculators_b200.convert.mtp.stitch import stitch


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description="Stitch finetuned MTP weights back into a verifier checkpoint")
    ap.add_argument("finetuned_checkpoint", type=Path, help="fine-tuned MTP speculator checkpoint directory")
    ap.add_argument("verifier_path", type=Path, help="verifier checkpoint directory or hub model id")
    ap.add_argument("--output-path", type=Path, default=None)
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(message)s")
    out = args.output_path or Path.cwd() / f"{args.verifier_path.name}-stitched"
    stitch(args.finetuned_checkpoint, args.verifier_path, out)
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
