"""End-to-end CPU runs of the train entry point: preprocessed dataset on disk, cached
hidden states through the file backend, checkpoints, resume."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

import speculators_b200 as sb
from speculators_b200.train.config import TrainConfig
from speculators_b200.train.entrypoint import create_transformer_layer_config, main

from conftest import TINY_VERIFIER


def _make_dataset(root, n=12, layers=4, H=64, vocab=128, seed=0):
    from datasets import Dataset

    g = torch.Generator().manual_seed(seed)
    rows = []
    for i in range(n):
        L = int(torch.randint(12, 40, (1,), generator=g))
        ids = torch.randint(0, vocab, (L,), generator=g).tolist()
        mask = [0] * 4 + [1] * (L - 4)
        rows.append({"input_ids": ids, "loss_mask": mask, "seq_len": L})
    Dataset.from_list(rows).save_to_disk(str(root))
    hs = root / "hidden_states"
    hs.mkdir()
    freq: dict[int, int] = {}
    for i, r in enumerate(rows):
        save_file({"hidden_states": torch.randn(r["seq_len"], layers, H, generator=g).to(torch.bfloat16),
                   "token_ids": torch.tensor(r["input_ids"])}, str(hs / f"hs_{i}.safetensors"))
        for t in r["input_ids"]:
            freq[t] = freq.get(t, 0) + 1
    torch.save(freq, root / "token_freq.pt")


def _argv(verifier, data, save, *extra):
    return ["--verifier-name-or-path", verifier, "--data-path", str(data), "--save-path", str(save), "--total-seq-len", "64",
            "--num-workers", "0", "--on-missing", "raise", "--optimizer", "adamw", "--lr", "1e-3", "--draft-vocab-size", "32",
            "--target-layer-ids", "1", "2", "3", "--train-data-ratio", "0.75", "--log-freq", "1", *extra]


def test_eagle3_train_checkpoint_and_resume(tiny_verifier_dir, tmp_path):
    data, save = tmp_path / "data", tmp_path / "ckpt"
    _make_dataset(data)
    main(TrainConfig.resolve(_argv(tiny_verifier_dir, data, save, "--epochs", "2", "--ttt-steps", "2")))
    for epoch in ("0", "1"):
        d = save / epoch
        assert {"config.json", "model.safetensors", "optimizer_state_dict.pt", "scheduler_state_dict.pt", "training_state.json",
                "train_command.txt"} <= set(os.listdir(d))
    assert (save / "epoch1_end").is_symlink() and (save / "checkpoint_best").is_symlink()
    assert (save / "run.yaml").exists() and (data / "d2t.npy").exists()
    cfg = json.loads((save / "1" / "config.json").read_text())
    assert cfg["speculators_model_type"] == "eagle3" and cfg["torch_dtype"] == "bfloat16" and cfg["draft_vocab_size"] == 32
    assert cfg["transformer_layer_config"]["layer_types"] == ["sliding_attention"]
    weights = load_file(str(save / "1" / "model.safetensors"))
    assert weights["fc.weight"].dtype == torch.bfloat16 and "layers.0.self_attn.q_proj.weight" in weights
    loaded = sb.SpeculatorModel.from_pretrained(str(save / "1"))
    assert isinstance(loaded, sb.Eagle3DraftModel)
    state = json.loads((save / "1" / "training_state.json").read_text())
    assert state["epoch"] == 1 and state["local_step"] == 0 and state["global_step"] > 0
    # resume: one more epoch continues the step counter
    main(TrainConfig.resolve(_argv(tiny_verifier_dir, data, save, "--epochs", "3", "--ttt-steps", "2")))
    state2 = json.loads((save / "2" / "training_state.json").read_text())
    assert state2["global_step"] > state["global_step"]
    # the re-loadable run.yaml reproduces the config
    again = TrainConfig.resolve(["--config", str(save / "run.yaml")])
    assert again.flatten()["draft_vocab_size"] == 32 and again.trainer.epochs == 3


@pytest.mark.parametrize("algo,extra", [
    ("dflash", ["--num-layers", "2", "--block-size", "4", "--max-anchors", "6", "--mask-token-id", "5"]),
    ("dspark", ["--block-size", "4", "--max-anchors", "6", "--mask-token-id", "5", "--markov-rank", "8"]),
    ("peagle", ["--num-depths", "3", "--mask-token-id", "5"]),
])
def test_other_algorithms_train_one_epoch(algo, extra, tiny_verifier_dir, tmp_path):
    data, save = tmp_path / "data", tmp_path / "ckpt"
    _make_dataset(data)
    main(TrainConfig.resolve(_argv(tiny_verifier_dir, data, save, "--speculator-type", algo, "--epochs", "1", "--max-steps", "2", *extra)))
    cfg = json.loads((save / "0" / "config.json").read_text())
    assert cfg["speculators_model_type"] == algo
    assert type(sb.SpeculatorModel.from_pretrained(str(save / "0"))).__name__.lower().startswith(algo.replace("peagle", "peagle"))


def test_dry_run_and_from_pretrained_config_only(tiny_verifier_dir, tmp_path):
    data, save = tmp_path / "data", tmp_path / "dry"
    _make_dataset(data, n=6)
    main(TrainConfig.resolve(_argv(tiny_verifier_dir, data, save, "--dry-run")))
    assert (save / "model.safetensors").exists() and not (save / "0").exists()
    os.remove(save / "model.safetensors")  # config-only directory -> fresh init from the saved config
    save2 = tmp_path / "ckpt2"
    argv = [a for a in _argv(tiny_verifier_dir, data, save2, "--from-pretrained", str(save), "--epochs", "1", "--max-steps", "1")]
    main(TrainConfig.resolve(argv))
    assert (save2 / "0" / "model.safetensors").exists()


def test_decoder_config_from_verifier(tiny_verifier_dir):
    cfg = create_transformer_layer_config(tiny_verifier_dir, 3, "llama", None, 128, [1])
    assert cfg.layer_types == ["sliding_attention", "full_attention", "sliding_attention"] and cfg.sliding_window == 128
    assert cfg.hidden_size == TINY_VERIFIER["hidden_size"] and cfg.num_hidden_layers == 3 and cfg.head_dim == 16
    with pytest.raises(ValueError):
        create_transformer_layer_config(tiny_verifier_dir, 2, "llama", None, 128, [5])
    with pytest.raises(ValueError):
        create_transformer_layer_config(tiny_verifier_dir, 2, "mamba", None, 128, [])


def test_in_job_online_mode_states_what_it_needs():
    """``--online-verifier-gpus`` refuses what it cannot do before touching a GPU."""
    from types import SimpleNamespace

    from speculators_b200.train.entrypoint import _run_online

    with pytest.raises(ValueError, match="eagle3 and peagle"):
        _run_online(SimpleNamespace(speculator_type="dflash", online_verifier_gpus=2), None, None, torch.bfloat16)
    with pytest.raises(ValueError, match="torchrun job of more than N ranks"):
        _run_online(SimpleNamespace(speculator_type="eagle3", online_verifier_gpus=2), None, None, torch.bfloat16)
    cfg = TrainConfig.resolve(["--verifier-name-or-path", "x", "--online-verifier-gpus", "4", "--online-ring-slots", "8"])
    flat = cfg.flatten()
    assert flat["online_verifier_gpus"] == 4 and flat["online_ring_slots"] == 8 and flat["online_timeout"] == 600.0
