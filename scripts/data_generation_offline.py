#!/usr/bin/env python3
"""Generate verifier hidden states ahead of training and store one safetensors file
per sample (``hs_<index>.safetensors``) next to the prepared dataset.

    python scripts/data_generation_offline.py --preprocessed-data ./training_data \\
        --endpoint http://localhost:8000/v1 --concurrency 32 --validate-outputs

The server must have been started for hidden-state extraction
(``scripts/launch_vllm.py``).  Runs are resumable (existing files are skipped) and can
be split across nodes with ``--world-size/--rank``.

CLI parity: scripts/data_generation_offline.py:58 (parse_args), :437 (main) of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import asyncio
import logging
import sys
from pathlib import Path

from speculators_b200.data_generation.offline import (
    OfflineRunConfig, get_existing_hidden_state_indices, get_indices_to_process, run_offline_generation,
)
from speculators_b200.data_generation.vllm_client import DEFAULT_MAX_RETRIES, DEFAULT_REQUEST_TIMEOUT, generate_hidden_states_async
from speculators_b200.train.data import build_client_item
from speculators_b200.train.logger import setup_root_logger

logger = logging.getLogger(__name__)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Generate draft-model training data offline")
    ap.add_argument("--model", default=None, help="expected served model id (checked against the endpoint)")
    ap.add_argument("--endpoint", default="http://localhost:8000/v1", help="OpenAI-compatible base URL of the server")
    ap.add_argument("--preprocessed-data", default="./output", help="dataset written by prepare_data.py")
    ap.add_argument("--max-samples", type=int, default=None)
    ap.add_argument("--output", default=None, help="default: <preprocessed-data>/hidden_states")
    ap.add_argument("--concurrency", type=int, default=32, help="requests kept in flight")
    ap.add_argument("--validate-outputs", action="store_true", help="reload every file; check token ids, length, finiteness")
    ap.add_argument("--request-timeout", type=float, default=DEFAULT_REQUEST_TIMEOUT)
    ap.add_argument("--max-retries", type=int, default=DEFAULT_MAX_RETRIES)
    ap.add_argument("--fail-on-error", action="store_true", help="abort on the first sample that fails after its retries")
    ap.add_argument("--max-consecutive-errors", type=int, default=None,
                    help="abort after this many failed samples in a row (default: --concurrency)")
    ap.add_argument("--world-size", type=int, default=1, help="number of NODES sharing the run")
    ap.add_argument("--rank", type=int, default=0, help="index of this node in [0, world-size)")
    return ap


async def generate(args: argparse.Namespace, dataset) -> int:
    import openai
    from tqdm import tqdm

    out_dir = Path(args.output) if args.output else Path(args.preprocessed_data) / "hidden_states"
    todo = get_indices_to_process(
        len(dataset), args.max_samples, get_existing_hidden_state_indices(out_dir), args.world_size, args.rank
    )
    if not todo:
        return 0
    logger.info("Processing %d samples", len(todo))
    cfg = OfflineRunConfig(
        output_dir=out_dir, concurrency=args.concurrency, validate_outputs=args.validate_outputs,
        request_timeout=args.request_timeout, max_retries=args.max_retries, fail_on_error=args.fail_on_error,
        max_consecutive_errors=None if args.fail_on_error else args.max_consecutive_errors,
    )
    async with openai.AsyncOpenAI(base_url=args.endpoint, api_key="EMPTY", max_retries=0) as client:
        served = (await client.models.list()).data[0].id
        if args.model and args.model != served:
            raise ValueError(f"--model {args.model} does not match the served model {served}; check --endpoint.")

        def item(idx: int) -> dict:
            row = dataset[idx]
            return dict(build_client_item(row))

        async def request(payload: dict) -> str:
            return await generate_hidden_states_async(client, served, payload, timeout=cfg.request_timeout, max_retries=cfg.max_retries)

        with tqdm(total=len(todo)) as bar:
            def progress(stats):
                bar.n = stats.ok + stats.errors
                bar.set_postfix({"ok": stats.ok, "err": stats.errors}, refresh=False)
                bar.refresh()

            stats = await run_offline_generation(todo, item, request, cfg, progress)
    logger.info("%s", stats.summary())
    if stats.skipped:
        logger.warning("Skipped %d samples due to errors: %s", len(stats.skipped), stats.skipped)
    return 0


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    """Parsed command line (``sys.argv`` when ``argv`` is None)."""
    return build_parser().parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if not 0 <= args.rank < args.world_size:
        raise ValueError("--rank must be in range [0, world_size)")
    setup_root_logger()
    from datasets import load_from_disk

    dataset = load_from_disk(args.preprocessed_data).with_format(None)
    try:
        asyncio.run(generate(args, dataset))
    except KeyboardInterrupt:
        return 130
    except Exception:
        logger.exception("Data generation failed")
        return 1
    logger.info("Data generation complete!")
    return 0


if __name__ == "__main__":
    sys.exit(main())
