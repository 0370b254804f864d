"""``python -m speculators_b200`` command line: ``--version`` and ``convert``
(src/speculators/__main__.py:77-183).  Built on argparse."""

from __future__ import annotations

import argparse
import json
import sys

from speculators_b200.version import __version__


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="speculators_b200", description="Speculators (B200-native) command line.")
    parser.add_argument("--version", action="version", version=f"speculators_b200 version: {__version__}")
    sub = parser.add_subparsers(dest="command")
    conv = sub.add_parser("convert", help="Convert an external draft checkpoint into the speculators format.")
    conv.add_argument("model", help="Checkpoint directory or hub id.")
    conv.add_argument("--verifier", required=True, help="Verifier model the draft belongs to.")
    conv.add_argument("--algorithm", required=True, choices=["eagle3", "mtp", "dflash"])
    conv.add_argument("--output-path", default="converted")
    conv.add_argument("--validate-device", default=None, help="Load the converted checkpoint once to validate it.")
    conv.add_argument("--algorithm-kwargs", default=None, help='JSON dict of converter options, e.g. \'{"norm_before_residual": true}\'.')
    return parser


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    if args.command != "convert":
        build_parser().print_help()
        return 0
    kwargs = {}
    if args.algorithm_kwargs:
        try:
            kwargs = json.loads(args.algorithm_kwargs)
        except json.JSONDecodeError as err:
            raise SystemExit(f"--algorithm-kwargs is not valid JSON: {err}") from err
        if not isinstance(kwargs, dict):
            raise SystemExit("--algorithm-kwargs must be a JSON object")
    from speculators_b200.convert.entrypoints import convert_model

    convert_model(args.model, verifier=args.verifier, algorithm=args.algorithm, output_path=args.output_path, validate_device=args.validate_device, **kwargs)
    return 0



def app(argv: list[str] | None = None) -> None:
    """Console entry point (the reference exposes its command line under this name)."""
    raise SystemExit(main(argv))


if __name__ == "__main__":
    sys.exit(main())
