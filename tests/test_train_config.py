"""Layered training configuration: flag > YAML > default, recorded per field; conflicts and
mismatches; the command-line boundary turns configuration errors into a clean exit(2)."""

import warnings

import pytest
import yaml
from pydantic import ValidationError

from speculators_b200.train.config import TrainConfig
from speculators_b200.train.config.resolution import ConfigError
from speculators_b200.train.config.schema import nest_flat


def _write(tmp_path, text):
    path = tmp_path / "run.yaml"
    path.write_text(text)
    return str(path)


def _src(cli, **kw):
    return TrainConfig.from_sources(cli=cli, argv=["train.py"], **kw)


def test_flag_beats_default_and_winning_layer_is_recorded():
    cfg = _src({"verifier_name_or_path": "some-model", "lr": 0.5})
    flat = cfg.flatten()
    assert flat["verifier_name_or_path"] == "some-model" and flat["lr"] == 0.5 and flat["epochs"] == 20
    assert cfg._provenance["lr"] == "flag" and cfg._provenance["epochs"] == "default"


def test_schema_violations_raise_from_the_pure_constructor():
    with pytest.raises(ValidationError):
        _src({"verifier_name_or_path": "m", "checkpoint_freq": 1.5})
    with pytest.raises(ValidationError):
        _src({"verifier_name_or_path": "m", "hidden_states_dtype": "float16"})
    with pytest.raises(ValidationError):
        _src({"verifier_name_or_path": "m", "hidden_states_dtype": "nn"})
    with pytest.raises(ConfigError, match="--verifier-name-or-path"):
        _src({})
    with pytest.raises(ConfigError, match="from-pretrained"):
        _src({"verifier_name_or_path": "m", "from_pretrained": "ckpt", "num_layers": 2})


def test_yaml_beats_default_and_flag_beats_yaml(tmp_path):
    path = _write(tmp_path, "train:\n  optimizer:\n    lr: 0.2\n  trainer:\n    epochs: 7\n")
    cfg = _src({"verifier_name_or_path": "m", "lr": 0.9}, config_path=path)
    flat = cfg.flatten()
    assert (flat["lr"], flat["epochs"], flat["weight_decay"]) == (0.9, 7, 0.01)
    assert (cfg._provenance["lr"], cfg._provenance["epochs"], cfg._provenance["weight_decay"]) == ("flag", "yaml", "default")


def test_layers_merge_inside_one_group(tmp_path):
    path = _write(tmp_path, "train:\n  optimizer:\n    weight_decay: 0.5\n")
    cfg = _src({"verifier_name_or_path": "m", "lr": 0.9}, config_path=path)
    assert cfg.flatten()["lr"] == 0.9 and cfg.flatten()["weight_decay"] == 0.5
    assert cfg._provenance["weight_decay"] == "yaml"


def test_yaml_shapes(tmp_path):
    cfg = _src({}, config_path=_write(tmp_path, "verifier:\n  verifier_name_or_path: from-bare\n"))
    assert cfg.flatten()["verifier_name_or_path"] == "from-bare" and cfg._provenance["verifier_name_or_path"] == "yaml"
    for contents in ("", "---\n", "# comment\n"):
        assert _src({"verifier_name_or_path": "m"}, config_path=_write(tmp_path, contents)).flatten()["verifier_name_or_path"] == "m"
    staged = "prepare_data:\n  data_path: ignored\nlaunch_vllm:\n  port: 8200\ntrain:\n  data:\n    data_path: from-train\n"
    assert _src({"verifier_name_or_path": "m"}, config_path=_write(tmp_path, staged)).flatten()["data_path"] == "from-train"


def test_unknown_keys_warn_and_valid_siblings_apply(tmp_path):
    path = _write(tmp_path, "train:\n  optimizer:\n    lr: 0.3\n    nonsense_knob: 1\n  bogus_group: {}\n")
    with pytest.warns(UserWarning, match="unrecognised keys"):
        cfg = _src({"verifier_name_or_path": "m"}, config_path=path)
    assert cfg.flatten()["lr"] == 0.3


def test_draft_init_conflicts_across_layers(tmp_path):
    with pytest.raises(ConfigError, match="from-pretrained"):
        _src({}, config_path=_write(tmp_path, "train:\n  draft:\n    from_pretrained: ckpt\n    num_layers: 4\n"))
    with pytest.raises(ConfigError, match="from-pretrained"):
        _src({"num_layers": 4}, config_path=_write(tmp_path, "train:\n  draft:\n    from_pretrained: ckpt\n"))
    with pytest.raises(ConfigError, match="from-pretrained"):
        _src({"from_pretrained": "ckpt"}, config_path=_write(tmp_path, "train:\n  draft:\n    num_layers: 4\n"))
    for cli in ({"from_pretrained": "ckpt"}, {"draft_config": "decoder"}, {"num_layers": 4, "draft_arch": "qwen3"}):
        assert _src({"verifier_name_or_path": "m", **cli}).speculator_type == "eagle3"


def test_every_scalar_flag_is_settable_via_yaml(tmp_path):
    probes = {dest: value for dest, value in TrainConfig().flatten().items() if isinstance(value, (int, float, str)) and not isinstance(value, bool)}
    probes["verifier_name_or_path"] = "m"
    cfg = _src({}, config_path=_write(tmp_path, yaml.safe_dump({"train": nest_flat(probes)})))
    for dest in probes:
        assert cfg._provenance[dest] == "yaml", dest


def test_algorithm_block_mismatch_warnings(tmp_path):
    with pytest.warns(UserWarning, match="does not use the 'dspark'"):
        _src({"verifier_name_or_path": "m", "markov_rank": 128})
    with pytest.warns(UserWarning, match="does not use the 'dflash'"):
        _src({"verifier_name_or_path": "m", "speculator_type": "peagle"}, config_path=_write(tmp_path, "train:\n  dflash:\n    block_size: 16\n"))
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        _src({"verifier_name_or_path": "m", "speculator_type": "dspark", "block_size": 16, "markov_rank": 128})
        _src({"verifier_name_or_path": "m", "speculator_type": "eagle3"})


def test_command_line_boundary_exits_cleanly(tmp_path, capsys):
    with pytest.raises(SystemExit) as exc:
        TrainConfig.resolve([])
    assert exc.value.code == 2 and "--verifier-name-or-path" in capsys.readouterr().err

    config = tmp_path / "ok.yaml"
    config.write_text("train:\n  verifier:\n    verifier_name_or_path: from-yaml\n  optimizer:\n    lr: 0.2\n")
    assert TrainConfig.resolve(["--config", str(config)]).flatten()["verifier_name_or_path"] == "from-yaml"
    assert TrainConfig.resolve(["--config", str(config), "--lr", "0.5"]).flatten()["lr"] == 0.5

    for argv in (["--verifier-name-or-path", "m", "--checkpoint-freq", "1.5"], ["--verifier-name-or-path", "m", "--hidden-states-dtype", "float16"]):
        with pytest.raises(SystemExit) as exc:
            TrainConfig.resolve(argv)
        err = capsys.readouterr().err
        assert exc.value.code == 2 and "invalid configuration" in err and "Traceback" not in err

    bad = tmp_path / "bad.yaml"
    bad.write_text("train:\n  optimizer:\n  lr: [unclosed\n")
    with pytest.raises(SystemExit) as exc:
        TrainConfig.resolve(["--verifier-name-or-path", "m", "--config", str(bad)])
    err = capsys.readouterr().err
    assert exc.value.code == 2 and str(bad) in err and "Traceback" not in err

    bad.write_text("- just\n- a\n- list\n")
    with pytest.raises(SystemExit) as exc:
        TrainConfig.resolve(["--verifier-name-or-path", "m", "--config", str(bad)])
    err = capsys.readouterr().err
    assert exc.value.code == 2 and "top-level mapping" in err and "Traceback" not in err


# ---------------------------------------------------------------- artifacts: run.yaml, --dump-config
def _resolved(**cli):
    with warnings.catch_warnings():
        warnings.filterwarnings("ignore", message=".*does not use the.*algorithm group.*", category=UserWarning)
        return TrainConfig.from_sources(cli=cli, config_path=None, argv=["train.py"])


def _reload(tmp_path, cfg):
    path = tmp_path / "run.yaml"
    path.write_text(cfg.dump_yaml())
    with warnings.catch_warnings():
        warnings.filterwarnings("ignore", message=".*does not use the.*algorithm group.*", category=UserWarning)
        return TrainConfig.from_sources(cli={}, config_path=str(path), argv=["train.py"])


@pytest.mark.parametrize("cli", [
    {"verifier_name_or_path": "m"},
    {"verifier_name_or_path": "m", "lr": 0.9, "num_layers": 4},
    {"verifier_name_or_path": "m", "from_pretrained": "ckpt"},
    {"verifier_name_or_path": "m", "speculator_type": "dspark", "markov_rank": 128},
    {"verifier_name_or_path": "m", "target_layer_ids": [2, 5, 9]},
    {"verifier_name_or_path": "m", "loss_fn": '{"ce": 0.1, "tv": 0.9}'},
])
def test_dumped_yaml_reloads_to_the_same_resolved_config(tmp_path, cli):
    cfg = _resolved(**cli)
    assert cfg.flatten() == _reload(tmp_path, cfg).flatten()


def test_dumped_yaml_is_stable_stage_wrapped_and_minimal(tmp_path):
    cfg = _resolved(verifier_name_or_path="m", lr=0.9, num_layers=4, epochs=7)
    assert _reload(tmp_path, cfg).dump_yaml() == cfg.dump_yaml()
    doc = yaml.safe_load(_resolved(verifier_name_or_path="m", lr=0.9).dump_yaml())
    assert doc == {"train": {"verifier": {"verifier_name_or_path": "m"}, "optimizer": {"lr": 0.9}}}


def test_save_writes_exactly_run_yaml_and_train_command(tmp_path):
    cfg = _resolved(verifier_name_or_path="m", num_layers=6, lr=0.3)
    cfg.save(str(tmp_path))
    assert {p.name for p in tmp_path.iterdir()} == {"run.yaml", "train_command.txt"}
    manifest = (tmp_path / "train_command.txt").read_text()
    assert "train.py" in manifest and "# Git SHA:" in manifest and "# World size:" in manifest
    reran = TrainConfig.from_sources(cli={}, config_path=str(tmp_path / "run.yaml"), argv=["train.py"])
    assert reran.flatten() == cfg.flatten()


def test_config_rebuilt_from_a_flat_dict_still_dumps(tmp_path):
    resolved = _resolved(verifier_name_or_path="m", speculator_type="eagle3", save_path="/tmp/ckpt", epochs=7, lr=0.3)
    rebuilt = TrainConfig.from_flat(resolved.flatten())
    assert rebuilt.provenance == {}
    doc = rebuilt.dump_yaml()
    assert "train:" in doc and "save_path" in doc and "/tmp/ckpt" in doc
    rebuilt.save(str(tmp_path))
    assert (tmp_path / "run.yaml").exists()


def test_dump_config_prints_a_reloadable_config_and_exits(tmp_path, capsys):
    with pytest.raises(SystemExit) as exc:
        TrainConfig.resolve(["--verifier-name-or-path", "m", "--lr", "0.5", "--num-layers", "7", "--dump-config"])
    assert exc.value.code == 0
    printed = capsys.readouterr().out
    doc = yaml.safe_load(printed)
    assert doc["train"]["optimizer"]["lr"] == 0.5 and doc["train"]["verifier"]["verifier_name_or_path"] == "m"
    path = tmp_path / "printed.yaml"
    path.write_text(printed)
    reran = TrainConfig.from_sources(cli={}, config_path=str(path), argv=["train.py"])
    assert reran.draft.num_layers == 7 and reran.verifier.verifier_name_or_path == "m"
    config = tmp_path / "run.yaml"
    config.write_text("train:\n  optimizer:\n    lr: 0.2\n")
    with pytest.raises(SystemExit):
        TrainConfig.resolve(["--verifier-name-or-path", "m", "--config", str(config), "--dump-config"])
    assert yaml.safe_load(capsys.readouterr().out)["train"]["optimizer"]["lr"] == 0.2


# ---------------------------------------------------------------- schema: flat <-> nested
def test_flatten_and_from_flat_are_inverse():
    cfg = TrainConfig()
    flat = cfg.flatten()
    assert TrainConfig.from_flat(flat).flatten() == flat
    assert TrainConfig.from_flat({**flat, "not_a_config_key": 1}).flatten() == flat  # foreign keys are ignored
    partial = TrainConfig.from_flat({"lr": 0.7, "verifier_name_or_path": "m"})
    assert partial.flatten()["lr"] == 0.7 and partial.flatten()["epochs"] == 20
    nested = nest_flat({"lr": 0.7, "epochs": 3})
    assert nested == {"optimizer": {"lr": 0.7}, "trainer": {"epochs": 3}}


def test_flatten_resolves_algorithm_dependent_defaults():
    e = TrainConfig.from_flat({"verifier_name_or_path": "m"}).flatten()
    assert (e["draft_arch"], e["norm_before_fc"], e["norm_output"], e["num_layers"], e["block_size"]) == ("llama", True, True, 1, 8)
    d = TrainConfig.from_flat({"verifier_name_or_path": "m", "speculator_type": "dflash"}).flatten()
    assert (d["draft_arch"], d["norm_before_fc"], d["norm_output"], d["num_layers"], d["block_size"], d["loss_fn"]) == ("qwen3", False, False, 5, 16, "ce")
    x = TrainConfig.from_flat({"verifier_name_or_path": "m", "speculator_type": "dflash", "num_layers": 2, "loss_fn": "kl_div",
                               "per_position_loss_weight": "fixed-exp-decay"}).flatten()
    assert (x["num_layers"], x["loss_fn"]) == (2, "kl_div")
    with pytest.raises(ValidationError, match="requires --loss-fn=ce"):  # the dflash default weighting needs cross-entropy
        TrainConfig.from_flat({"verifier_name_or_path": "m", "speculator_type": "dflash", "loss_fn": "kl_div"})


def test_help_lists_flags_grouped_by_concern():
    from speculators_b200.train.config.resolution import build_parser

    titles = {group.title for group in build_parser()._action_groups}
    assert {"general", "verifier", "draft", "data", "optimizer", "mtp"} <= titles
