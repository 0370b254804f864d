#!/usr/bin/env python3
"""Split SPEED-Bench flat files (``<config>.jsonl`` as written by the benchmark's own
``prepare.py``) into one JSONL per category (``qualitative``) or per
entropy/sub-category (``throughput_*``), each with a single ``turns`` column — the form
``evaluate.py --dataset speedbench/...`` consumes.

    python prepare_speedbench.py --data-dir ./speedbench_data [--configs qualitative,throughput_1k] [--download]

``--download`` first fetches and runs the upstream ``prepare.py`` (it materialises
prompts from third-party sources with their own licences: do not redistribute the
resulting files).  CLI parity: scripts/evaluate/prepare_speedbench.py:143 of the reference.
"""

from __future__ import annotations

import argparse
import json
import logging
import subprocess
import sys
import urllib.request
from pathlib import Path

logger = logging.getLogger("prepare_speedbench")

ALL_CONFIGS = ("qualitative", "throughput_1k", "throughput_2k", "throughput_8k", "throughput_32k")
PLACEHOLDERS = ("FULL BENCHMARK DATA SHOULD BE FETCHED FROM THE SOURCE", "{article}")
UPSTREAM_PREPARE = "https://raw.githubusercontent.com/NVIDIA-NeMo/Skills/refs/heads/main/nemo_skills/dataset/speed-bench/prepare.py"


class PlaceholderError(RuntimeError):
    pass


def prompt_text(row: dict) -> str:
    """``turns`` if present, else the first message's content (first turn only)."""
    if row.get("turns"):
        return row["turns"]
    msgs = row.get("messages") or []
    return msgs[0].get("content", "") if msgs else ""


def _slug(value: str | None) -> str:
    return (value or "unknown").replace(" ", "_").replace("/", "_")


def split_config(flat_file: Path, out_dir: Path, config: str) -> int:
    buckets: dict[str, list[str]] = {}
    with flat_file.open() as fh:
        for line in fh:
            if not line.strip():
                continue
            row = json.loads(line)
            text = prompt_text(row)
            if not text:
                continue
            if any(mark in text for mark in PLACEHOLDERS):
                raise PlaceholderError(f"Placeholder text in {config}/{row.get('category', '?')}: run the upstream prepare.py first.")
            key = _slug(row.get("category"))
            if config != "qualitative":
                key += "__" + _slug(row.get("sub_category"))
            buckets.setdefault(key, []).append(text)
    for key, texts in sorted(buckets.items()):
        with (out_dir / f"{config}_{key}.jsonl").open("w") as fh:
            fh.writelines(json.dumps({"turns": t}) + "\n" for t in texts)
        logger.info("  wrote %s_%s.jsonl (%d rows)", config, key, len(texts))
    return len(buckets)


def _run_upstream_prepare(data_dir: Path, configs: list[str]) -> None:
    with urllib.request.urlopen(UPSTREAM_PREPARE) as resp:  # noqa: S310
        script = resp.read()
    for config in configs:
        subprocess.run([sys.executable, "-", "--config", config, "--output_dir", str(data_dir)], input=script, check=True)  # noqa: S603


def main(argv: list[str] | None = None) -> int:
    logging.basicConfig(level=logging.INFO, format="[%(levelname)s] %(message)s")
    ap = argparse.ArgumentParser(description="Split SPEED-Bench flat files into per-category JSONL files.")
    ap.add_argument("--data-dir", required=True, type=Path)
    ap.add_argument("--configs", default=",".join(ALL_CONFIGS))
    ap.add_argument("--download", action="store_true", help="fetch and run the upstream prepare.py first")
    args = ap.parse_args(argv)
    args.data_dir.mkdir(parents=True, exist_ok=True)
    configs = [c.strip() for c in args.configs.split(",") if c.strip()]
    if args.download:
        _run_upstream_prepare(args.data_dir, configs)
    total = 0
    for config in configs:
        flat = args.data_dir / f"{config}.jsonl"
        if not flat.exists():
            logger.warning("Skipping %s: %s not found.", config, flat)
            continue
        try:
            total += split_config(flat, args.data_dir, config)
        except PlaceholderError as err:
            logger.error("%s", err)
            return 1
    logger.info("Done. %d files written to %s", total, args.data_dir)
    return 0


if __name__ == "__main__":
    sys.exit(main())
