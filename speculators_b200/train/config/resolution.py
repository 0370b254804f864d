"""From ``argv`` + optional YAML to a validated ``TrainConfig``.

* ``build_parser`` generates the argparse CLI from the schema: ``Literal`` ->
  ``choices``, ``list[T]`` -> ``nargs='+'``, bools that default to True / None (or
  are tagged) -> ``--x/--no-x``, other bools -> ``store_true``; every default is
  ``SUPPRESS`` so only flags the user typed are seen.  Hidden-state backends
  contribute their own flags, carried outside the schema.
* ``build_from_sources`` deep-merges ``flag > yaml > default``, records which layer
  supplied each value, then applies the cross-field rules: exactly one way to
  define the draft (``--from-pretrained`` | ``--draft-config`` | decoder-shaping
  flags; MTP reuses the verifier's decoder), required values, warnings for
  algorithm blocks the chosen speculator type ignores.
* ``resolve`` is the only function that touches ``sys.argv`` / exits: any
  configuration error becomes ``SystemExit(2)``; ``--dump-config`` prints the
  resolved ``run.yaml`` and exits 0.

Behavioural parity: src/speculators/train/config/resolution.py:120-573.
"""

from __future__ import annotations

import argparse
import sys
import types
import typing
import warnings
from pathlib import Path
from typing import Any, Literal, Union

import yaml
from pydantic import ValidationError

from speculators_b200.hs_connectors import HiddenStatesBackend
from speculators_b200.train.config.schema import CONFIG_DESTS, DEST_TO_GROUP, GROUPS, ROOT_FIELDS, TrainConfig, nest_flat

__all__ = ["BACKEND_DESTS", "ConfigError", "add_config_cli_arguments", "build_from_sources", "build_parser", "resolve"]


class ConfigError(ValueError):
    """A configuration mistake the user can fix (rendered without a traceback)."""


def _flag(dest: str) -> str:
    return "--" + dest.replace("_", "-")


DECODER_SHAPING_FLAGS: dict[str, str] = {
    d: _flag(d) for d in ("num_layers", "draft_arch", "draft_hidden_act", "sliding_window", "full_attention_indices")
}
_ALGORITHM_GROUP_USERS: dict[str, frozenset[str]] = {
    "dflash": frozenset({"dflash", "dspark"}), "dspark": frozenset({"dspark"}),
    "peagle": frozenset({"peagle"}), "mtp": frozenset({"mtp"}),
}
_CHOICE_REGISTRIES: dict[str, Any] = {"hidden_states_backends": HiddenStatesBackend.registry}


def _all_fields() -> dict[str, Any]:
    fields = {name: TrainConfig.model_fields[name] for name in ROOT_FIELDS}
    for gmodel in GROUPS.values():
        fields.update(gmodel.model_fields)
    return fields


REQUIRED_FLAGS: dict[str, str] = {
    dest: _flag(dest) for dest, f in _all_fields().items()
    if isinstance(f.json_schema_extra, dict) and f.json_schema_extra.get("cli_required")
}


# ---- backend-contributed flags -------------------------------------------------------------
def _collect_backend_args():
    per_backend: dict[str, list[argparse.Action]] = {}
    owner: dict[str, str] = {}
    for name, backend in sorted(HiddenStatesBackend.registry.items()):
        scratch = argparse.ArgumentParser(add_help=False)
        backend.add_train_args(scratch)
        actions = [a for a in scratch._actions if a.dest not in ("help", argparse.SUPPRESS)]  # noqa: SLF001
        per_backend[name] = actions
        for action in actions:
            if action.dest in owner:
                raise RuntimeError(f"Backend '{name}' and '{owner[action.dest]}' both register train-arg dest '{action.dest}'")
            if action.dest in CONFIG_DESTS:
                raise RuntimeError(f"Backend '{name}' train-arg dest '{action.dest}' collides with an existing schema field")
            owner[action.dest] = name
    return per_backend, frozenset(owner)


_BACKEND_ACTIONS, BACKEND_DESTS = _collect_backend_args()
_BACKEND_DESTS = BACKEND_DESTS  # the reference's name


def _backfill_backend_defaults(backend: str, merged: dict[str, Any]) -> None:
    for action in _BACKEND_ACTIONS.get(backend, []):
        if action.dest not in merged and action.default is not argparse.SUPPRESS:
            merged[action.dest] = action.default


# ---- schema -> argparse --------------------------------------------------------------------
def _annotation_spec(annotation: Any) -> tuple[Any, bool, list[Any] | None]:
    """-> (element type, is_list, choices) with ``Optional`` stripped."""
    origin = typing.get_origin(annotation)
    if origin in (Union, types.UnionType):
        inner = [a for a in typing.get_args(annotation) if a is not type(None)]
        if len(inner) == 1:
            return _annotation_spec(inner[0])
    if origin is Literal:
        values = list(typing.get_args(annotation))
        return type(values[0]), False, values
    if origin in (list, typing.List):  # noqa: UP006
        (elem,) = typing.get_args(annotation) or (str,)
        base, _, choices = _annotation_spec(elem)
        return base, True, choices
    return annotation, False, None


def _add_field_argument(target, dest: str, field) -> None:  # noqa: ANN001
    base, is_list, choices = _annotation_spec(field.annotation)
    extra = field.json_schema_extra if isinstance(field.json_schema_extra, dict) else {}
    registry_key = extra.get("cli_choices")
    if registry_key:
        choices = sorted(_CHOICE_REGISTRIES[registry_key])
    kwargs: dict[str, Any] = {"dest": dest, "default": argparse.SUPPRESS, "help": field.description}
    if base is bool:
        default = field.default
        if default is True or default is None or extra.get("cli_bool") == "optional":
            kwargs["action"] = argparse.BooleanOptionalAction
        else:
            kwargs["action"] = "store_true"
    else:
        kwargs["type"] = base if base in (int, float, str) else str
        if is_list:
            kwargs["nargs"] = "+"
        if choices:
            kwargs["choices"] = choices
    target.add_argument(_flag(dest), **kwargs)


def add_config_cli_arguments(parser: argparse.ArgumentParser) -> None:
    """One flag per schema field; ``--help`` lists them grouped by concern (``general`` for
    the root fields, then one argparse group per config group)."""
    general = parser.add_argument_group("general")
    for name in ROOT_FIELDS:
        _add_field_argument(general, name, TrainConfig.model_fields[name])
    for gname, gmodel in GROUPS.items():
        group = parser.add_argument_group(gname)
        for dest, field in gmodel.model_fields.items():
            _add_field_argument(group, dest, field)
    for actions in _BACKEND_ACTIONS.values():
        for action in actions:
            kwargs = {"dest": action.dest, "default": argparse.SUPPRESS, "help": action.help}
            if action.type is not None:
                kwargs["type"] = action.type
            if action.choices is not None:
                kwargs["choices"] = action.choices
            if action.nargs is not None:
                kwargs["nargs"] = action.nargs
            parser.add_argument(*action.option_strings, **kwargs)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Train a speculative-decoding draft model.")
    parser.add_argument("--config", dest="config", default=None, metavar="PATH",
                        help="YAML config (trainer keys under a top-level 'train:' key; a bare mapping is accepted). Flags override it.")
    parser.add_argument("--dump-config", dest="dump_config", action="store_true",
                        help="Print the fully resolved config as a run.yaml and exit.")
    add_config_cli_arguments(parser)
    return parser


# ---- YAML ----------------------------------------------------------------------------------
def _load_config_file(path: str) -> dict[str, Any]:
    try:
        data = yaml.safe_load(Path(path).read_text())
    except OSError as exc:
        raise ConfigError(f"--config '{path}' could not be read: {exc.strerror or exc}") from exc
    except yaml.YAMLError as exc:
        raise ConfigError(f"--config '{path}' is not valid YAML: {exc}") from exc
    if data is None:
        return {}
    if not isinstance(data, dict):
        raise ConfigError(f"--config '{path}' must contain a top-level mapping.")
    return data


def _unwrap_stage(data: dict[str, Any]) -> dict[str, Any]:
    stage = data.get("train")
    return stage if isinstance(stage, dict) else data


def _partition_yaml_keys(nested: dict[str, Any]) -> tuple[set[str], set[str]]:
    known: set[str] = set()
    unknown: set[str] = set()
    for key, value in nested.items():
        if key in GROUPS and isinstance(value, dict):
            for leaf in value:
                (known if leaf in GROUPS[key].model_fields else unknown).add(leaf)
        elif key == "backend" and isinstance(value, dict):
            for leaf in value:
                (known if leaf in BACKEND_DESTS else unknown).add(leaf)
        elif key in ROOT_FIELDS:
            known.add(key)
        else:
            unknown.add(key)
    return known, unknown


def _deep_merge(base: dict[str, Any], top: dict[str, Any]) -> dict[str, Any]:
    out = dict(base)
    for key, value in top.items():
        if isinstance(value, dict) and isinstance(out.get(key), dict):
            out[key] = _deep_merge(out[key], value)
        else:
            out[key] = value
    return out


# ---- cross-field rules -----------------------------------------------------------------------
def _reject(conflicting: list[str], reason: str) -> None:
    if conflicting:
        raise ConfigError(f"{reason} (remove them): {', '.join(conflicting)}")


def _validate_draft_init(cfg: TrainConfig, provided: set[str]) -> None:
    shaping = [flag for dest, flag in DECODER_SHAPING_FLAGS.items() if dest in provided]
    with_config = shaping + (["--draft-config"] if cfg.draft.draft_config else [])
    if cfg.draft.from_pretrained:
        _reject(with_config, "--from-pretrained loads a complete draft model and takes precedence over all other model-definition options, so these conflict with it")
    elif cfg.speculator_type == "mtp":
        _reject(with_config, "--speculator-type mtp reuses the verifier's decoder config, so these options do not apply")
    elif cfg.draft.draft_config:
        _reject(shaping, "--draft-config defines the draft decoder, so these flags conflict with it")


def _warn_mismatched_algorithm_blocks(cfg: TrainConfig, provided: set[str]) -> None:
    for group, users in _ALGORITHM_GROUP_USERS.items():
        if cfg.speculator_type in users:
            continue
        ignored = sorted(_flag(d) for d in GROUPS[group].model_fields if d in provided)
        if ignored:
            warnings.warn(
                f"--speculator-type {cfg.speculator_type} does not use the '{group}' algorithm group; these settings are "
                f"ignored: {', '.join(ignored)}", stacklevel=2,
            )


def _validate_required(cfg: TrainConfig) -> None:
    for dest, flag in REQUIRED_FLAGS.items():
        if cfg.provenance[dest] == "default":
            raise ConfigError(f"missing required value: set {flag} or provide it in --config")


def build_from_sources(cls: type[TrainConfig], *, cli: dict[str, Any], config_path: str | None, argv: list[str],
                       backend_cli: dict[str, Any] | None = None) -> TrainConfig:
    yaml_nested: dict[str, Any] = {}
    yaml_dests: set[str] = set()
    if config_path is not None:
        yaml_nested = _unwrap_stage(_load_config_file(config_path))
        yaml_dests, unknown = _partition_yaml_keys(yaml_nested)
        if unknown:
            warnings.warn(f"--config '{config_path}' has unrecognised keys (ignored): {', '.join(sorted(unknown))}", stacklevel=2)
    schema_yaml = {k: v for k, v in yaml_nested.items() if k in GROUPS or k in ROOT_FIELDS}
    cfg = cls(**_deep_merge(schema_yaml, nest_flat(cli)))
    cfg._provenance = {d: ("flag" if d in cli else "yaml" if d in yaml_dests else "default") for d in CONFIG_DESTS}
    cfg._argv = list(argv)
    yaml_backend = {k: v for k, v in (yaml_nested.get("backend") or {}).items() if k in BACKEND_DESTS} if isinstance(yaml_nested.get("backend"), dict) else {}
    merged = {**yaml_backend, **(backend_cli or {})}
    _backfill_backend_defaults(cfg.data.hidden_states_backend, merged)
    cfg._backend_args = merged
    for dest in BACKEND_DESTS:
        if backend_cli and dest in backend_cli:
            cfg._provenance[dest] = "flag"
        elif dest in yaml_backend:
            cfg._provenance[dest] = "yaml"
    provided = {d for d, layer in cfg._provenance.items() if layer != "default"}
    _warn_mismatched_algorithm_blocks(cfg, provided)
    _validate_draft_init(cfg, provided)
    _validate_required(cfg)
    return cfg


def _format_validation_error(exc: ValidationError) -> str:
    lines = []
    for err in exc.errors():
        where = ".".join(str(p) for p in err["loc"]) or "<config>"
        lines.append(f"{where}: {err['msg'].removeprefix('Value error, ')}")
    return "invalid configuration:\n  " + "\n  ".join(lines)


def resolve(cls: type[TrainConfig], argv: list[str] | None) -> TrainConfig:
    parser = build_parser()
    ns = vars(parser.parse_args(argv))
    cli = {d: v for d, v in ns.items() if d in CONFIG_DESTS}
    backend_cli = {d: v for d, v in ns.items() if d in BACKEND_DESTS}
    full_argv = list(sys.argv) if argv is None else [sys.argv[0], *argv]
    try:
        cfg = cls.from_sources(cli=cli, config_path=ns["config"], argv=full_argv, backend_cli=backend_cli)
    except ValidationError as exc:
        parser.error(_format_validation_error(exc))
    except ConfigError as exc:
        parser.error(str(exc))
    if ns["dump_config"]:
        sys.stdout.write(cfg.dump_yaml())
        raise SystemExit(0)
    return cfg
