#!/usr/bin/env python3
"""Start a vLLM server that exports verifier hidden states.

    python scripts/launch_vllm.py MODEL [--hidden-states-backend file|mooncake]
        [--target-layer-ids 2 16 29] [--dry-run] -- <extra vllm serve arguments>

Builds the ``--speculative_config`` (``extract_hidden_states`` with the auxiliary layer
ids; default ``[2, L//2, L-3]`` plus the last layer ``L``) and the
``--kv_transfer_config`` of the chosen transfer backend, then replaces this process with
``vllm serve``.

CLI parity: scripts/launch_vllm.py:50 (parse_args), :107 (main) of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import json
import os
import sys
import warnings

from speculators_b200.hs_connectors import HiddenStatesBackend


def build_parser() -> argparse.ArgumentParser:
    backends = HiddenStatesBackend.registry
    ap = argparse.ArgumentParser(
        description="Launch vLLM for hidden states extraction",
        usage="launch_vllm.py [-h] MODEL [--hidden-states-backend BACKEND] [--target-layer-ids ID [ID ...]] -- *VLLM_ARGS",
    )
    ap.add_argument("model", help="model name or path to extract hidden states from")
    ap.add_argument("--hidden-states-backend", choices=sorted(backends), default="file")
    for backend in backends.values():  # every backend contributes its own flags
        backend.add_launch_args(ap)
    ap.add_argument("--target-layer-ids", type=int, nargs="+",
                    help="layer ids to export; the same list must be given to training")
    ap.add_argument("--include-last-layer", action=argparse.BooleanOptionalAction, default=True,
                    help="also export the final layer (verifier logits are recomputed from it)")
    ap.add_argument("--dry-run", action="store_true", help="print the command instead of running it")
    ap.add_argument("--trust-remote-code", action="store_true",
                    help="allow custom config code when resolving layer ids (pass it again after '--' for vLLM)")
    return ap


def resolve_layer_ids(num_hidden_layers: int, requested: list[int] | None, include_last: bool) -> list[int]:
    if not requested:
        return [2, num_hidden_layers // 2, num_hidden_layers - 3, num_hidden_layers]
    ids = list(requested)
    if include_last and num_hidden_layers not in ids:
        ids.append(num_hidden_layers)
    warnings.warn(f"Using custom target layer ids {ids}. These must also be passed to the training script.", stacklevel=2)
    return ids


def build_command(args: argparse.Namespace, vllm_args: list[str], num_hidden_layers: int) -> list[str]:
    layer_ids = resolve_layer_ids(num_hidden_layers, args.target_layer_ids, args.include_last_layer)
    spec_cfg = {
        "method": "extract_hidden_states",
        "num_speculative_tokens": 1,
        "draft_model_config": {"hf_config": {"eagle_aux_hidden_state_layer_ids": layer_ids}},
    }
    kv_cfg = HiddenStatesBackend.registry[args.hidden_states_backend].build_kv_transfer_config(args)
    return [
        sys.executable, "-m", "vllm.entrypoints.cli.main", "serve", args.model,
        "--speculative_config", json.dumps(spec_cfg), "--kv_transfer_config", json.dumps(kv_cfg), *vllm_args,
    ]


def _num_hidden_layers(model: str, trust_remote_code: bool) -> int:
    from transformers import AutoConfig

    cfg = AutoConfig.from_pretrained(model, trust_remote_code=trust_remote_code)
    return getattr(cfg, "text_config", cfg).num_hidden_layers


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    """Parsed command line (``sys.argv`` when ``argv`` is None)."""
    return build_parser().parse_args(argv)


def main(argv: list[str] | None = None) -> int:
    args, vllm_args = build_parser().parse_known_args(argv)
    if "--" in vllm_args:
        vllm_args.remove("--")
    cmd = build_command(args, vllm_args, _num_hidden_layers(args.model, args.trust_remote_code))
    print("Running command:")
    print(" ".join(cmd))
    if not args.dry_run:
        os.execvp(cmd[0], cmd)  # noqa: S606
    return 0


if __name__ == "__main__":
    sys.exit(main())
