"""Trainer-side helpers: train_command.txt, validation re-synchronisation, dataset splits,
rotary settings of the derived draft config."""

import json
import os
import sys
from types import SimpleNamespace
from unittest.mock import patch

import pytest

from speculators_b200.train import trainer as trainer_mod
from speculators_b200.train.trainer import Trainer
from speculators_b200.train.utils import save_train_command


# ---------------------------------------------------------------- train_command.txt
def test_train_command_file_has_header_and_quoted_command(tmp_path):
    target = tmp_path / "nested" / "dir"
    with patch.object(sys, "argv", ["scripts/train.py", "--lr", "1e-4", "--path", "/has spaces/dir"]), \
            patch.dict(os.environ, {"WORLD_SIZE": "8"}):
        save_train_command(str(target))
    text = (target / "train_command.txt").read_text()
    assert "# Timestamp:" in text and "# Git SHA:" in text and "# World size: 8" in text
    for pkg in ("speculators_b200", "transformers", "torch"):
        assert f"# {pkg}:" in text
    assert text.rstrip().splitlines()[-1] == "scripts/train.py --lr 1e-4 --path '/has spaces/dir'"
    assert [f for f in os.listdir(target) if f != "train_command.txt"] == []  # no temporary file left behind


def test_train_command_defaults_and_overwrite(tmp_path):
    (tmp_path / "train_command.txt").write_text("old content")
    env = {k: v for k, v in os.environ.items() if k != "WORLD_SIZE"}
    with patch.dict(os.environ, env, clear=True), patch("speculators_b200.provenance.find_repo_root", return_value=None):
        save_train_command(str(tmp_path), argv=["train.py", "--epochs", "3"])
    text = (tmp_path / "train_command.txt").read_text()
    assert "old content" not in text and "# World size: 1" in text and "# Git SHA: unknown" in text
    assert text.rstrip().endswith("train.py --epochs 3")


# ---------------------------------------------------------------- validation re-sync
def _barrier_indices(n_batches, *, is_distributed, interval):
    stand_in = SimpleNamespace(is_distributed=is_distributed, config=SimpleNamespace(process_group=None))
    hit = []
    with patch.object(trainer_mod, "_VAL_SYNC_INTERVAL", interval), patch.object(trainer_mod.dist, "barrier") as barrier:
        for i in range(n_batches):
            before = barrier.call_count
            Trainer._maybe_val_sync(stand_in, i)
            if barrier.call_count > before:
                hit.append(i)
    return hit


def test_validation_barriers_only_on_interval_boundaries():
    assert _barrier_indices(200, is_distributed=True, interval=50) == [50, 100, 150]
    assert 0 not in _barrier_indices(10, is_distributed=True, interval=1)
    assert _barrier_indices(200, is_distributed=False, interval=50) == []
    assert _barrier_indices(200, is_distributed=True, interval=0) == []


@pytest.mark.parametrize("interval", [1, 7, 50, 500])
def test_every_rank_reaches_the_same_number_of_barriers(interval):
    n = 1864
    a = _barrier_indices(n, is_distributed=True, interval=interval)
    assert a == _barrier_indices(n, is_distributed=True, interval=interval) and len(a) == (n - 1) // interval


# ---------------------------------------------------------------- dataset splits
def _arrow_dir(tmp_path, n):
    from datasets import Dataset

    ds = Dataset.from_dict({"input_ids": [[i, i + 1, i + 2] for i in range(n)], "loss_mask": [[1, 1, 1]] * n, "seq_len": [3] * n})
    path = tmp_path / "data"
    ds.save_to_disk(str(path))
    (path / "hidden_states").mkdir()
    return str(path)


@pytest.mark.parametrize("ratio", [0.1, 0.25, 0.3, 0.7, 0.95])
@pytest.mark.parametrize("n", [1000, 12501])
def test_train_and_val_splits_are_exactly_complementary(tmp_path, ratio, n):
    from speculators_b200.train.data import ArrowDataset

    path = _arrow_dir(tmp_path, n)
    train = ArrowDataset(max_len=128, datapath=path, on_missing="skip", train_ratio=ratio, split="train")
    val = ArrowDataset(max_len=128, datapath=path, on_missing="skip", train_ratio=ratio, split="val")
    assert len(train) + len(val) == n and len(train) == int(n * ratio)
    first_val = val.data[0]["input_ids"][0] if hasattr(val, "data") else None
    if first_val is not None:
        assert first_val == len(train)  # val starts right where train stops


def test_split_argument_validation(tmp_path):
    from speculators_b200.train.data import ArrowDataset

    path = _arrow_dir(tmp_path, 10)
    with pytest.raises(ValueError, match="train_ratio"):
        ArrowDataset(max_len=128, datapath=path, on_missing="skip", train_ratio=1.5)
    with pytest.raises(ValueError, match="validation"):
        ArrowDataset(max_len=128, datapath=path, on_missing="skip", train_ratio=1.0, split="val")
    with pytest.raises(ValueError, match="empty"):
        ArrowDataset(max_len=128, datapath=path, on_missing="skip", train_ratio=0.01, split="train")


# ---------------------------------------------------------------- rotary settings of the draft
def _verifier_dir(tmp_path, name="verifier", **overrides):
    cfg = {"model_type": "qwen3", "vocab_size": 1000, "hidden_size": 512, "num_attention_heads": 8, "num_key_value_heads": 8,
           "intermediate_size": 2048, "max_position_embeddings": 4096, "initializer_range": 0.02, "rms_norm_eps": 1e-6,
           "hidden_act": "silu", "head_dim": 64, "num_hidden_layers": 4, "rope_theta": 10000.0}
    cfg.update(overrides)
    d = tmp_path / name
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    return str(d)


def _draft(vdir, **kw):
    from speculators_b200.train.entrypoint import create_transformer_layer_config

    args = dict(verifier_name_or_path=vdir, num_layers=1, draft_arch="llama", hidden_act="silu", sliding_window=0, full_attention_indices=[])
    args.update(kw)
    return create_transformer_layer_config(**args)


def test_draft_keeps_mrope_sections_and_drops_the_legacy_type_alias(tmp_path):
    rope = {"type": "default", "rope_type": "default", "mrope_section": [8, 12, 12], "mrope_interleaved": True, "rope_theta": 500000.0}
    cfg = _draft(_verifier_dir(tmp_path, rope_scaling=rope))
    kept = cfg.rope_parameters
    assert kept["mrope_section"] == [8, 12, 12] and "type" not in kept and "mrope_interleaved" not in kept
    assert kept["rope_theta"] == 500000.0 and cfg.rope_theta == 500000.0


def test_partial_rotary_mrope_is_expanded_to_the_full_head(tmp_path):
    rope = {"rope_type": "default", "mrope_section": [4, 6, 6], "partial_rotary_factor": 0.5}
    cfg = _draft(_verifier_dir(tmp_path, rope_parameters=rope))
    assert cfg.rope_parameters["mrope_section"] == [8, 12, 12] and cfg.rope_parameters["partial_rotary_factor"] == 1.0
    kept = _draft(_verifier_dir(tmp_path, "b", rope_parameters=rope), mrope_full_head_hack=False)
    assert kept.rope_parameters["mrope_section"] == [4, 6, 6]
    with pytest.raises(ValueError, match="not an integer"):
        _draft(_verifier_dir(tmp_path, "c", rope_parameters=dict(rope, partial_rotary_factor=0.3)))


def test_plain_rope_scaling_is_carried_without_partial_factor(tmp_path):
    rope = {"rope_type": "llama3", "factor": 8.0, "partial_rotary_factor": 0.5}
    cfg = _draft(_verifier_dir(tmp_path, rope_scaling=rope), full_attention_indices=[0])
    assert cfg.rope_parameters["rope_type"] == "llama3" and "partial_rotary_factor" not in cfg.rope_parameters
    assert cfg.layer_types == ["full_attention"]
    with pytest.raises(ValueError, match="Full attention indices"):
        _draft(_verifier_dir(tmp_path, "d"), full_attention_indices=[3])
