"""Data preparation, offline generation, MTP stitching, benchmark harness and launch
helpers: CPU tests with fakes for the server side."""

import argparse
import asyncio
import importlib.util
import json
import sys
from pathlib import Path

import pytest
import torch
from safetensors.torch import load_file, save_file

from speculators_b200.data_generation import preprocessing as pp
from speculators_b200.data_generation.offline import ConsecutiveFailureAbort, OfflineRunConfig, run_offline_generation

ROOT = Path(__file__).resolve().parent.parent


def _script(name):
    spec = importlib.util.spec_from_file_location(f"script_{name}", ROOT / "scripts" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


class CharTemplate:
    """Toy chat template: ``<role>`` marker token, one token per character, ``;`` closes a
    turn; the generation prompt is the assistant marker.  ``scaffold`` pre-fills a
    thinking tag in the generation prompt (as reasoning templates do)."""

    ROLES = {"system": 1, "user": 2, "assistant": 3, "tool": 4}

    def __init__(self, scaffold=False, drop_history_reasoning=False):
        self.scaffold = scaffold
        self.calls = 0

    def __call__(self, messages, *, add_generation_prompt, tools=None):
        self.calls += 1
        ids = [9, len(tools)] if tools else []
        for m in messages:
            ids.append(self.ROLES[m["role"]])
            if m.get("reasoning_content"):
                ids += [7] + [100 + ord(c) for c in m["reasoning_content"]] + [8]
            ids += [100 + ord(c) for c in m["content"]] + [5]
        if add_generation_prompt:
            ids.append(3)
            if self.scaffold:
                ids += [7, 8]
        return ids


def test_normalize_and_adapt():
    conv = [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "yo", "thinking": "hm"},
            {"role": "my-model", "content": "x"}, {"role": "tool", "content": "r", "tool_call_id": "c1"}]
    norm = pp.normalize_conversation(conv)
    assert [t["role"] for t in norm] == ["user", "assistant", "assistant", "tool"]
    assert norm[1]["reasoning_content"] == "hm" and norm[3]["tool_call_id"] == "c1"
    wire = pp.adapt_conversation_for_server([{"role": "user", "content": ["a", {"type": "image", "path": "/x/y.png"}]}])
    assert wire[0]["content"][0] == {"type": "text", "text": "a"}
    assert wire[0]["content"][1] == {"type": "image_url", "image_url": {"url": "file:///x/y.png"}}


def test_boundary_rows_one_per_assistant_turn():
    conv = pp.normalize_conversation([{"role": "user", "content": "ab"}, {"role": "assistant", "content": "cd"},
                                      {"role": "user", "content": "e"}, {"role": "assistant", "content": "fgh"},
                                      {"role": "user", "content": "trailing"}])
    rows = pp.boundary_rows(conv, CharTemplate(), 1000)
    assert len(rows) == 2
    first, second = rows
    # context = [user a b ;] + assistant marker; supervised = "cd;"
    assert first["loss_mask"] == [0] * 5 + [1] * 3 and len(first["input_ids"]) == 8
    assert sum(second["loss_mask"]) == 4 and second["loss_mask"][-4:] == [1] * 4
    assert len(second["conv"]) == 4
    # a turn whose context alone fills the window is skipped, later rows are not
    assert len(pp.boundary_rows(conv, CharTemplate(), 6)) == 1


def test_boundary_rows_scaffold_falls_back_to_common_prefix():
    conv = pp.normalize_conversation([{"role": "user", "content": "q"}, {"role": "assistant", "content": "a", "thinking": "t"}])
    rows = pp.boundary_rows(conv, CharTemplate(scaffold=True), 1000)
    # prompt = [2 q ; 3 7 8], full = [2 q ; 3 7 t 8 a ;] -> shared prefix of 5 tokens
    assert rows[0]["loss_mask"] == [0] * 5 + [1] * 4

    class Unstable(CharTemplate):
        def __call__(self, messages, *, add_generation_prompt, tools=None):
            ids = super().__call__(messages, add_generation_prompt=add_generation_prompt, tools=tools)
            return ([50] if len(messages) > 1 else [51]) + ids  # history changes once a turn is appended

    with pytest.raises(pp.BoundaryUnstableError):
        pp.boundary_rows(conv, Unstable(), 1000)


def test_preprocess_batch_paths():
    render = CharTemplate()
    batch = {"conversations": [
        [{"from": "human", "value": "hello"}, {"from": "gpt", "value": "world"}],
        None,
        [{"from": "human", "value": "only user"}],
        [{"from": "human", "value": "x"}, {"from": "gpt", "value": "yz"}, {"from": "human", "value": "w"}, {"from": "gpt", "value": "v"}],
    ], "tools": ['[{"name": "f"}]', None, "not json", None]}
    out = pp.preprocess_batch(batch, False, render, max_length=64, minimum_valid_tokens=2)
    assert len(out["input_ids"]) == 3 and out["seq_len"] == [len(x) for x in out["input_ids"]]
    assert out["input_ids"][0][:2].tolist() == [9, 1]  # tools were parsed and rendered for the first conversation
    assert all(int(m.sum()) >= 2 for m in out["loss_mask"])
    # clipping past the boundary drops the row as unsupervised
    out = pp.preprocess_batch({"conversations": batch["conversations"][:1]}, False, render, max_length=6)
    assert out["input_ids"] == []
    # pre-tokenised rows pass through; skew is an error
    out = pp.preprocess_batch({"input_ids": [[1, 2, 3, 4], [5, 6]], "loss_mask": [[0, 1, 1, 1], [0, 0]]}, False, None, 3)
    assert [t.tolist() for t in out["input_ids"]] == [[1, 2, 3]] and out["loss_mask"][0].tolist() == [0, 1, 1]
    with pytest.raises(ValueError, match="shape mismatch"):
        pp.preprocess_batch({"input_ids": [[1, 2]], "loss_mask": [[1]]}, False, None, 8)
    with pytest.raises(ValueError, match="renderer"):
        pp.preprocess_batch({"conversations": batch["conversations"]}, False, None, 8)


def test_build_dataset_and_load_raw(tmp_path):
    from datasets import Dataset

    path = tmp_path / "conv.jsonl"
    rows = [{"conversations": [{"from": "human", "value": f"q{i}"}, {"from": "gpt", "value": f"answer{i}"}]} for i in range(5)]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    raw, norm = pp.load_raw_dataset(str(path))
    assert norm is None and len(raw) == 5
    (tmp_path / "dir").mkdir()
    (tmp_path / "dir" / "a.jsonl").write_text(path.read_text())
    assert len(pp.load_raw_dataset(str(tmp_path / "dir"))[0]) == 5
    with pytest.raises(ValueError, match="Unsupported dataset"):
        pp.load_raw_dataset("nope")
    with pytest.raises(ValueError, match="Invalid hf: spec"):
        pp.load_raw_dataset("hf:a:b:c:d")
    built = pp.build_speculator_training_dataset(raw, object(), 64, num_proc=1, renderer=CharTemplate())
    assert len(built) == 5 and set(built.column_names) == {"input_ids", "loss_mask", "seq_len"}
    with pytest.raises(ValueError, match="render_endpoint is required"):
        pp.build_speculator_training_dataset(raw, object(), 64, num_proc=1)
    pre = Dataset.from_list([{"input_ids": [1, 2, 3], "loss_mask": [0, 1, 1]}])
    assert len(pp.build_speculator_training_dataset(pre, object(), 64, num_proc=1)) == 1


def test_render_client_error_policy(monkeypatch):
    from speculators_b200.data_generation import render_client as rc
    from speculators_b200.data_generation.vllm_client import InvalidResponseError

    replies = []
    monkeypatch.setattr(rc, "_post_json", lambda url, body, timeout: replies.pop(0))
    monkeypatch.setattr("time.sleep", lambda s: None)
    replies[:] = [(503, "busy"), (200, json.dumps({"token_ids": [1, 2]}))]
    assert rc.render_conversation("http://h:1/", [], add_generation_prompt=True) == [1, 2]
    replies[:] = [(404, "nope"), (200, "{}")]
    with pytest.raises(InvalidResponseError):
        rc.render_conversation("http://h:1", [], add_generation_prompt=False)
    assert len(replies) == 1  # not retried
    replies[:] = [(200, "{}")] * 2
    with pytest.raises(rc.RenderError, match="token_ids"):
        rc.render_conversation("http://h:1", [], add_generation_prompt=False, max_retries=1)


def test_prepare_data_overwrite_guard(tmp_path):
    mod = _script("prepare_data")
    out = tmp_path / "out"
    out.mkdir()
    for name in ("data-00000.arrow", "state.json", "token_freq.pt"):
        (out / name).write_text("x")
    mod.assert_safe_to_overwrite(out, out / "token_freq.pt")
    (out / "thesis.tex").write_text("mine")
    with pytest.raises(ValueError, match="thesis.tex"):
        mod.assert_safe_to_overwrite(out, out / "token_freq.pt")
    # an existing dataset is kept without --overwrite
    assert mod.main(["--model", "m", "--data", "d", "--output", str(out)]) == 0


def test_build_vocab_mapping_script(tmp_path):
    import numpy as np

    mod = _script("build_vocab_mapping")
    torch.save({3: 10, 7: 5, 1: 1}, tmp_path / "token_freq.pt")
    assert mod.main(["--token-freq-path", str(tmp_path / "token_freq.pt"), "--draft-vocab-size", "2", "--target-vocab-size", "10",
                     "--output-path", str(tmp_path)]) == 0
    t2d, d2t = np.load(tmp_path / "t2d.npy"), np.load(tmp_path / "d2t.npy")
    assert t2d.sum() == 2 and t2d[3] and t2d[7] and (np.arange(2) + d2t).tolist() == [3, 7]


def test_launch_vllm_command():
    mod = _script("launch_vllm")
    args, rest = mod.build_parser().parse_known_args(["some/model", "--hidden-states-path", "/data/hs", "--", "--tensor-parallel-size", "2"])
    rest.remove("--")
    cmd = mod.build_command(args, rest, 32)
    spec_cfg = json.loads(cmd[cmd.index("--speculative_config") + 1])
    assert spec_cfg["draft_model_config"]["hf_config"]["eagle_aux_hidden_state_layer_ids"] == [2, 16, 29, 32]
    kv = json.loads(cmd[cmd.index("--kv_transfer_config") + 1])
    assert kv["kv_connector_extra_config"]["shared_storage_path"] == "/data/hs" and cmd[-2:] == ["--tensor-parallel-size", "2"]
    with pytest.warns(UserWarning):
        assert mod.resolve_layer_ids(32, [1, 5], True) == [1, 5, 32]
        assert mod.resolve_layer_ids(32, [1, 5], False) == [1, 5]


def test_offline_runner(tmp_path):
    src = tmp_path / "server"
    src.mkdir()

    def make_item(idx):
        return {"input_ids": [idx, idx + 1, idx + 2]}

    async def request(item):
        idx = item["input_ids"][0]
        await asyncio.sleep(0.001)
        if idx % 5 == 4:
            raise TimeoutError("server busy")
        path = src / f"req_{idx}.safetensors"
        save_file({"token_ids": torch.tensor(item["input_ids"]), "hidden_states": torch.randn(3, 2, 4)}, str(path))
        return str(path)

    cfg = OfflineRunConfig(output_dir=tmp_path / "out", concurrency=3, validate_outputs=True, max_consecutive_errors=3)
    stats = asyncio.run(run_offline_generation(list(range(10)), make_item, request, cfg))
    assert stats.ok == 8 and stats.errors == 2 and sorted(stats.skipped) == [4, 9]
    assert sorted(p.name for p in (tmp_path / "out").iterdir()) == sorted(f"hs_{i}.safetensors" for i in range(10) if i % 5 != 4)
    assert "8 samples" in stats.summary()

    async def down(item):
        raise ConnectionError("refused")

    with pytest.raises(ConsecutiveFailureAbort):
        asyncio.run(run_offline_generation(list(range(10)), make_item, down, cfg))
    with pytest.raises(ConnectionError):
        asyncio.run(run_offline_generation([0, 1], make_item, down, OfflineRunConfig(output_dir=tmp_path / "o2", fail_on_error=True)))


def test_stitch_mtp_roundtrip(tmp_path):
    from speculators_b200.convert.mtp.converter import MTPConverter
    from speculators_b200.convert.mtp.stitch import native_key, stitch, unfuse_moe_experts

    g = torch.Generator().manual_seed(0)
    E, H, I = 3, 8, 4
    native = {"mtp.fc.weight": torch.randn(H, 2 * H, generator=g), "mtp.norm.weight": torch.randn(H, generator=g),
              "mtp.layers.0.self_attn.q_proj.weight": torch.randn(H, H, generator=g)}
    for e in range(E):
        for name, shape in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            native[f"mtp.layers.0.mlp.experts.{e}.{name}.weight"] = torch.randn(*shape, generator=g)
    body = {"model.embed_tokens.weight": torch.randn(16, H, generator=g), "lm_head.weight": torch.randn(16, H, generator=g)}
    verifier = tmp_path / "verifier"
    verifier.mkdir()
    save_file(body, str(verifier / "model-00001-of-00002.safetensors"))
    save_file(native, str(verifier / "model-00002-of-00002.safetensors"))
    wm = {k: "model-00001-of-00002.safetensors" for k in body} | {k: "model-00002-of-00002.safetensors" for k in native}
    (verifier / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    (verifier / "config.json").write_text("{}")
    # draft checkpoint: converted names, packed experts, every tensor shifted by +1 ("training")
    draft = MTPConverter.fuse_moe_experts({MTPConverter.remap_key(k): v + 1 for k, v in native.items()})
    draft["embed_tokens.weight"] = body["model.embed_tokens.weight"] + 5  # frozen: must be ignored
    assert any(k.endswith("experts.gate_up_proj") for k in draft)
    ckpt = tmp_path / "draft"
    ckpt.mkdir()
    save_file({k: v.contiguous() for k, v in draft.items()}, str(ckpt / "model.safetensors"))
    out = stitch(ckpt, verifier, tmp_path / "stitched")
    got = load_file(str(out / "model-00002-of-00002.safetensors"))
    assert set(got) == set(native)
    for k, v in native.items():
        torch.testing.assert_close(got[k], v + 1)
    untouched = load_file(str(out / "model-00001-of-00002.safetensors"))
    torch.testing.assert_close(untouched["model.embed_tokens.weight"], body["model.embed_tokens.weight"])
    assert (out / "config.json").exists()
    assert native_key(MTPConverter.remap_key("mtp.layers.0.mlp.gate.weight")) == "mtp.layers.0.mlp.gate.weight"
    with pytest.raises(ValueError, match="missing down_proj"):
        unfuse_moe_experts({"a.experts.gate_up_proj": torch.zeros(2, 4, 3)})
    bad = tmp_path / "bad"
    bad.mkdir()
    save_file({"mtp_layers.0.unknown.weight": torch.zeros(1)}, str(bad / "model.safetensors"))
    with pytest.raises(ValueError, match="not found in verifier weight map"):
        stitch(bad, verifier, tmp_path / "s2")


def test_benchmark_run_and_compare(tiny_verifier_dir, tmp_path, capsys):
    from speculators_b200.train import benchmark as bm
    from speculators_b200.train.config import TrainConfig

    torch.save({i: 100 - i for i in range(64)}, tmp_path / "token_freq.pt")
    train_argv = ["--verifier-name-or-path", tiny_verifier_dir, "--total-seq-len", "48", "--draft-vocab-size", "32",
                  "--target-layer-ids", "1", "2", "3", "--token-freq-path", str(tmp_path / "token_freq.pt"), "--ttt-steps", "2",
                  "--save-path", str(tmp_path / "unused"), "--data-path", str(tmp_path / "data")]
    results = {}
    for name, steps in (("a", 3), ("b", 4)):
        bench_args = argparse.Namespace(synthetic=True, warmup_steps=1, measured_steps=steps, output=str(tmp_path / f"{name}.json"), no_per_step=False)
        results[name] = bm.run_benchmark(bench_args, argparse.Namespace(**TrainConfig.resolve(train_argv).flatten()))
    a = json.loads((tmp_path / "a.json").read_text())
    assert a["benchmark_version"] == bm.BENCHMARK_VERSION and a["config"]["synthetic_data"] and a["config"]["num_target_layers"] == 3
    assert a["timing"]["step_ms"]["count"] == 3 and len(a["per_step"]) == 3 and a["timing"]["tokens_per_s"]["mean"] > 0
    assert set(a["timing"]) == set(bm.TIMING_KEYS) and "git_sha" in a["provenance"]
    report = bm.compare_benchmarks(str(tmp_path / "a.json"), str(tmp_path / "b.json"))
    assert "step_ms" in report and "peak_allocated_mb" in report and "COMPARABILITY" not in report
    b = results["b"]
    b["config"]["total_seq_len"] = 96
    assert "Sequence length: 48 vs 96" in bm.format_comparison(a, b)
    assert _script("benchmark").main(["compare", str(tmp_path / "a.json"), str(tmp_path / "b.json")]) == 0
