#!/usr/bin/env python3
"""Regenerate the assistant side of a dataset with the target model (on-policy data).

    python script.py --dataset ultrachat --endpoint http://127.0.0.1:8000/v1/chat/completions \\
        --limit 1000 --concurrency 64 --sampling-params '{"temperature": 0.6, "top_p": 0.95}'

Writes JSONL rows with ``input_ids`` / ``loss_mask`` (one per generation) that
``scripts/prepare_data.py`` takes as they are.  ``--resume`` skips conversations already
in the output file.  CLI parity: scripts/response_regeneration/script.py:62 of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import asyncio
import json
import logging
import os
import sys

from speculators_b200.data_generation import regeneration as rg
from speculators_b200.data_generation.configs import DATASET_CONFIGS
from speculators_b200.data_generation.vllm_client import DEFAULT_MAX_RETRIES, InvalidResponseError, with_retries

# the helpers live in the package; they are reachable from the script module too, under the
# names the reference script gives them
extract_conversation, extract_tools, load_seen = rg.extract_conversation, rg.extract_tools, rg.load_seen
regenerate_conversation, build_boundary_sample = rg.regenerate_conversation, rg.boundary_sample
_primary_identifier, prepare_row = rg.primary_identifier, rg.prepare_row

logger = logging.getLogger(__name__)
RETRYABLE_HTTP_STATUSES = frozenset({408, 409, 425, 429})


def _dataset_choice(name: str) -> str:
    if name in rg.MULTIMODAL_DATASETS:
        raise argparse.ArgumentTypeError(
            f"{name} is multimodal and regeneration does not support images (it is text-only). Generate its responses elsewhere and convert them with prepare_data.py."
        )
    return name


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Regenerate dataset responses via a Chat Completions endpoint.")
    ap.add_argument("--endpoint", default="http://127.0.0.1:8000/v1/chat/completions")
    ap.add_argument("--model", default=None, help="served model name (auto-detected when omitted)")
    ap.add_argument("--dataset", default="ultrachat", type=_dataset_choice, choices=rg.REGEN_DATASETS)
    ap.add_argument("--split", default=None)
    ap.add_argument("--subset", default=None)
    ap.add_argument("--limit", type=int, default=None, help="stop after N rows")
    ap.add_argument("--concurrency", type=int, default=64, help="conversations in flight")
    ap.add_argument("--max-tokens", type=int, default=8192)
    ap.add_argument("--sampling-params", default=None, help="JSON object merged into every request")
    ap.add_argument("--outfile", default=None)
    ap.add_argument("--resume", action="store_true", help="skip conversations already in the output file")
    ap.add_argument("--language-filter", default=None, help="only rows whose language field equals this")
    ap.add_argument("--max-retries", type=int, default=DEFAULT_MAX_RETRIES)
    ap.add_argument("--no-text", action="store_true", help="do not load the tokenizer / write the decoded review text")
    return ap


def parse_args(argv=None) -> argparse.Namespace:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.max_retries < 0:
        ap.error("--max-retries must be >= 0")
    try:
        args.sampling_params = json.loads(args.sampling_params) if args.sampling_params else {}
    except json.JSONDecodeError as err:
        ap.error(f"--sampling-params is not valid JSON: {err}")
    if not isinstance(args.sampling_params, dict):
        ap.error("--sampling-params must be a JSON object")
    return args


def iter_items(dataset, config, *, limit, language, seen):
    taken = 0
    for idx, row in enumerate(dataset):
        if limit is not None and taken >= limit:
            return
        if language and row.get("language") != language:
            continue
        try:
            item = rg.prepare_item(row, config, idx)
        except ValueError as err:
            logger.warning("Skipping row %d: %s", idx, err)
            continue
        if item is None or item["primary_id"] in seen:
            continue
        taken += 1
        yield item


async def amain(args: argparse.Namespace) -> int:
    import aiohttp
    from datasets import load_dataset
    from tqdm import tqdm

    config = DATASET_CONFIGS[args.dataset]
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None)) as session:
        model = args.model
        if model is None:
            async with session.get(args.endpoint.replace("/v1/chat/completions", "/v1/models")) as resp:
                models = (await resp.json()).get("data", [])
            if not models:
                raise ValueError("No models found at endpoint; pass --model")
            model = models[0]["id"]
            print(f"Auto-detected model: {model}")
        detok = None
        if not args.no_text:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(model)
            detok = lambda ids: tok.decode(ids, skip_special_tokens=False)  # noqa: E731
        outfile = args.outfile or f"{args.dataset}_{rg.sanitize_filename(model)}.jsonl"
        os.makedirs(os.path.dirname(os.path.abspath(outfile)), exist_ok=True)
        seen = rg.load_seen(outfile) if args.resume else set()
        dataset = load_dataset(config.hf_path, name=args.subset or config.subset, split=args.split or config.split, streaming=True)

        @with_retries
        async def post_once(payload: dict) -> dict:
            async with session.post(args.endpoint, json=payload) as resp:
                if resp.ok:
                    return await resp.json()
                text = f"HTTP {resp.status} from {args.endpoint}: {(await resp.text())[:500]}"
                if resp.status >= 500 or resp.status in RETRYABLE_HTTP_STATUSES:
                    raise RuntimeError(text)  # transient: retried with back-off
                raise InvalidResponseError(text)  # permanent: fails fast

        with open(outfile, "a" if args.resume else "w", encoding="utf-8") as fh, tqdm(total=args.limit) as bar:
            def write(row: dict) -> None:
                fh.write(json.dumps(row, ensure_ascii=False) + "\n")
                fh.flush()

            def tick(stats: rg.RegenStats) -> None:
                bar.update(1)
                bar.set_postfix({"ok": stats.ok, "err": stats.errors, "cut": stats.truncated}, refresh=False)

            stats = await rg.run_regeneration(
                iter_items(dataset, config, limit=args.limit, language=args.language_filter, seen=seen),
                lambda payload: post_once(payload, max_retries=args.max_retries), write, model=model, max_tokens=args.max_tokens,
                concurrency=args.concurrency, endpoint=args.endpoint, sampling_params=args.sampling_params, detokenize=detok, on_done=tick,
            )
    print("\n" + stats.summary())
    print(f"Output: {outfile}")
    return 0


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(message)s")
    return asyncio.run(amain(parse_args(argv)))


if __name__ == "__main__":
    sys.exit(main())
