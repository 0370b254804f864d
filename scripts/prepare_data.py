#!/usr/bin/env python3
"""Prepare on-policy data for draft-model training.

Inputs are conversations whose assistant turns were produced by the target model
(``.json``/``.jsonl`` files, directories, preset names, ``hf:`` specs) or rows that
already hold ``input_ids`` and ``loss_mask``.  Conversations are tokenised by the target
model's server (``--render-endpoint``) and masked at every assistant-turn boundary.
Outputs: an Arrow dataset in ``--output`` and the token-frequency table
(``token_freq.pt``) used to pick the draft vocabulary.  An existing dataset in
``--output`` is kept unless ``--overwrite`` is given.

    python scripts/prepare_data.py --model meta-llama/Llama-3.1-8B-Instruct \\
        --data ./on_policy.jsonl --render-endpoint http://localhost:8000 --output ./training_data

CLI parity: scripts/prepare_data.py:83 (parse_args), :206 (main) of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import logging
import shutil
import sys
from pathlib import Path

from speculators_b200.data_generation.logging_utils import PipelineLogger
from speculators_b200.data_generation.preprocessing import load_and_preprocess_dataset

log = PipelineLogger(__name__)

# what this script itself writes into --output; --overwrite deletes nothing else
OWN_ARTIFACT_NAMES = frozenset({"dataset_info.json", "state.json", "token_freq.pt"})


def foreign_files(output: Path, token_freq_path: Path) -> list[Path]:
    """Entries of ``output`` that are not artifacts of this script."""
    freq = token_freq_path.resolve()
    own = lambda p: p.is_file() and (p.suffix == ".arrow" or p.name in OWN_ARTIFACT_NAMES or p.resolve() == freq)  # noqa: E731
    return [p for p in output.iterdir() if not own(p)]


def assert_safe_to_overwrite(output: Path, token_freq_path: Path) -> None:
    extra = foreign_files(output, token_freq_path)
    if extra:
        raise ValueError(
            "--overwrite would delete files that do not look like prepare_data.py artifacts: "
            + ", ".join(map(str, extra)) + ". Remove them manually or choose a different --output directory."
        )


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Prepare data for speculator training")
    ap.add_argument("--model", required=True, help="target model id or path (its processor / chat template is used)")
    ap.add_argument("--trust-remote-code", action="store_true", help="allow custom code when loading the processor")
    ap.add_argument("--data", action="append", required=True,
                    help="on-policy conversations or input_ids/loss_mask rows; repeatable")
    ap.add_argument("--seq-length", type=int, default=8192, help="rows are clipped to this many tokens (default 8192)")
    ap.add_argument("--max-samples", type=int, default=None, help="cap on the number of rows written")
    ap.add_argument("--token-freq-path", default=None, help="default: <output>/token_freq.pt")
    ap.add_argument("--render-endpoint", default=None,
                    help="base URL of the target model's server, e.g. http://localhost:8000 (no /v1 suffix: "
                         "/v1/chat/completions/render is appended). Required unless all inputs are pre-tokenised.")
    ap.add_argument("--output", default="./output", help="dataset directory (default ./output)")
    ap.add_argument("--overwrite", action="store_true", help="re-run and replace this script's artifacts in --output")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--num-preprocessing-workers", type=int, default=8)
    ap.add_argument("--minimum-valid-tokens", type=int, default=None, help="drop rows with fewer supervised tokens")
    ap.add_argument("--allow-empty-output", action="store_true", help="do not fail when every row was filtered out")
    return ap


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    """Parsed command line (``sys.argv`` when ``argv`` is None)."""
    return build_parser().parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s - %(name)s - %(levelname)s - %(message)s")
    args = build_parser().parse_args(argv)
    out = Path(args.output)
    freq = Path(args.token_freq_path) if args.token_freq_path else out / "token_freq.pt"
    log.section("Preparing data")
    log.config({"Target Model": args.model, "Dataset": args.data, "Output Dir": args.output})
    if out.exists():
        if not args.overwrite and any(out.glob("*.arrow")):
            log.warning("Dataset files already exist in the output directory, skipping preprocessing (use --overwrite to redo).")
            return 0
        if args.overwrite:
            assert_safe_to_overwrite(out, freq)
            log.warning(f"Removing existing output directory: {out}")
            shutil.rmtree(out)
    out.mkdir(parents=True, exist_ok=True)
    dataset, _ = load_and_preprocess_dataset(
        args.model, args.data, seq_length=args.seq_length, build_dataset_num_proc=args.num_preprocessing_workers,
        seed=args.seed, max_samples=args.max_samples, token_freq_path=freq, render_endpoint=args.render_endpoint,
        minimum_valid_tokens=args.minimum_valid_tokens, allow_empty_output=args.allow_empty_output,
        trust_remote_code=args.trust_remote_code,
    )
    log.section(f"Writing dataset to {args.output}")
    dataset.save_to_disk(args.output)
    return 0


if __name__ == "__main__":
    sys.exit(main())
