"""Small utilities: rank filter of the logger, pydantic class registry, checkpoint loading helpers."""

import json
import logging

import pytest
import torch
from pydantic import BaseModel
from safetensors.torch import save_file

from speculators_b200.train.logger import IsRank0Filter
from speculators_b200.utils import loading
from speculators_b200.utils.pydantic_utils import PydanticClassRegistryMixin, ReloadableBaseModel


def _record(**extra):
    record = logging.LogRecord("speculators", logging.INFO, __file__, 0, "msg", None, None)
    for k, v in extra.items():
        setattr(record, k, v)
    return record


def test_rank0_filter_uses_the_global_rank(monkeypatch):
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("LOCAL_RANK", "0")  # first process of a second node: not global rank 0
    assert IsRank0Filter().filter(_record()) is False
    monkeypatch.setenv("RANK", "0")
    assert IsRank0Filter().filter(_record()) is True
    monkeypatch.setenv("RANK", "3")
    assert IsRank0Filter().filter(_record(override_rank0_filter=True)) is True


# ---------------------------------------------------------------- pydantic registry
def test_reloadable_model_and_registry_marshalling():
    class Plain(ReloadableBaseModel):
        x: int = 1

    assert Plain().x == 1
    Plain.reload_schema()  # must not raise
    assert Plain(x=3).model_dump() == {"x": 3}

    class Shape(PydanticClassRegistryMixin):
        schema_discriminator = "kind"
        kind: str

        @classmethod
        def __pydantic_schema_base_type__(cls):
            return Shape if cls.__name__ == "Shape" else cls

    @Shape.register("circle")
    class Circle(Shape):
        kind: str = "circle"
        r: float = 1.0

    @Shape.register()
    class Square(Shape):
        kind: str = "Square"
        side: float = 2.0

    assert Shape.registry["circle"] is Circle and "Square" in Shape.registry
    with pytest.raises(TypeError):
        Shape.register_decorator(object)  # not a pydantic model

    class Holder(BaseModel):
        shape: Shape

    Shape.reload_schema()
    Holder.model_rebuild(force=True)
    held = Holder.model_validate({"shape": {"kind": "circle", "r": 2.5}})
    assert isinstance(held.shape, Circle) and held.shape.r == 2.5
    assert isinstance(Shape.model_validate({"kind": "Square"}), Square)
    assert Holder.model_validate(held.model_dump()).shape == held.shape


# ---------------------------------------------------------------- loading helpers
def test_config_only_dir_detection(tmp_path):
    assert not loading.is_config_only_dir(tmp_path)  # no config.json
    (tmp_path / "config.json").write_text("{}")
    assert loading.is_config_only_dir(tmp_path)
    for name in ("pytorch_model.bin", "model.safetensors.index.json", "pytorch_model.bin.index.json", "model-00001-of-00002.safetensors"):
        marker = tmp_path / name
        marker.write_text("x")
        assert not loading.is_config_only_dir(tmp_path), name
        marker.unlink()
    assert not loading.is_config_only_dir(tmp_path / "config.json")  # a file, not a directory


def test_key_resolution_exact_suffix_and_aliases():
    keys = ["model.embed_tokens.weight", "model.layers.0.mlp.up_proj.weight", "output.weight", "norm.weight"]
    assert loading._match("model.embed_tokens.weight", keys) == "model.embed_tokens.weight"
    assert loading._match("embed_tokens.weight", keys) == "model.embed_tokens.weight"  # suffix
    assert loading._match("lm_head.weight", keys) == "output.weight"  # alias, exact
    assert loading._match("model.norm.weight", keys) == "norm.weight"
    assert loading._match("llm.embed.weight", ["prefix.llm.embed.weight"]) == "prefix.llm.embed.weight"
    assert loading._match("missing.weight", keys) is None
    assert loading._match("lm_head.weight", ["lm_head.weight", "output.weight"]) == "lm_head.weight"  # exact beats alias


def test_load_layers_from_single_file_and_sharded_checkpoints(tmp_path):
    tensors = {"model.embed_tokens.weight": torch.randn(8, 4), "model.norm.weight": torch.randn(4), "lm_head.weight": torch.randn(8, 4)}
    single = tmp_path / "single"
    single.mkdir()
    save_file(tensors, str(single / "model.safetensors"))
    got = loading.load_model_layers(["embed_tokens.weight", "lm_head.weight", "nope.weight"], single)
    assert set(got) == {"embed_tokens.weight", "lm_head.weight"}
    assert torch.equal(got["embed_tokens.weight"], tensors["model.embed_tokens.weight"])
    assert sorted(loading.list_checkpoint_keys(single)) == sorted(tensors)

    sharded = tmp_path / "sharded"
    sharded.mkdir()
    save_file({"model.embed_tokens.weight": tensors["model.embed_tokens.weight"]}, str(sharded / "a.safetensors"))
    save_file({k: v for k, v in tensors.items() if k != "model.embed_tokens.weight"}, str(sharded / "b.safetensors"))
    wmap = {"model.embed_tokens.weight": "a.safetensors", "model.norm.weight": "b.safetensors", "lm_head.weight": "b.safetensors"}
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wmap}))
    got = loading.load_model_layers(["model.norm.weight", "embed_tokens.weight"], sharded)
    assert torch.equal(got["model.norm.weight"], tensors["model.norm.weight"]) and torch.equal(got["embed_tokens.weight"], tensors["model.embed_tokens.weight"])
    with pytest.raises(ValueError, match="None of the requested"):
        loading.load_model_layers(["nope.weight"], sharded)
    with pytest.raises(FileNotFoundError):
        loading.list_checkpoint_keys(tmp_path)


def test_provenance_helpers(tmp_path):
    import subprocess

    from speculators_b200 import provenance

    lines = provenance.package_versions()
    assert all(line.startswith("# ") and ": " in line for line in lines)
    assert provenance.package_versions(("definitely-not-a-package",)) == ["# definitely-not-a-package: not installed"]
    assert provenance.git_sha(None) == "unknown" and provenance.git_diff(None) == ""
    assert provenance.run_git(["git", "rev-parse", "HEAD"], tmp_path) == ""  # not a repository
    assert provenance.find_package_repo("no_such_package_anywhere") is None
    repo = tmp_path / "repo"
    repo.mkdir()
    env = {"GIT_AUTHOR_NAME": "t", "GIT_AUTHOR_EMAIL": "t@t", "GIT_COMMITTER_NAME": "t", "GIT_COMMITTER_EMAIL": "t@t", "PATH": __import__("os").environ["PATH"]}
    subprocess.run(["git", "init", "-q"], cwd=repo, check=True, env=env)
    (repo / "a.txt").write_text("one\n")
    subprocess.run(["git", "add", "a.txt"], cwd=repo, check=True, env=env)
    subprocess.run(["git", "commit", "-q", "-m", "first"], cwd=repo, check=True, env=env)
    sha = provenance.git_sha(repo)
    assert len(sha) == 40 and provenance.git_diff(repo) == ""
    (repo / "a.txt").write_text("two\n")
    assert "+two" in provenance.git_diff(repo)
    assert provenance.find_repo_root(repo / "a.txt") == repo
    provenance.atomic_write(repo / "sub" / "f.txt", "hello")
    assert (repo / "sub" / "f.txt").read_text() == "hello" and [p.name for p in (repo / "sub").iterdir()] == ["f.txt"]


def test_ptxas_info_parser():
    from speculators_b200.ops._build import parse_ptxas_info

    text = """ptxas info    : 0 bytes gmem
ptxas info    : Compiling entry function '_ZN5sb2001aEv' for 'sm_100a'
ptxas info    : Function properties for _ZN5sb2001aEv
    48 bytes stack frame, 44 bytes spill stores, 40 bytes spill loads
ptxas info    : Used 168 registers, used 10 barriers, 48 bytes cumulative stack size, 1024 bytes smem
ptxas info    : Compile time = 10.0 ms
ptxas info    : Compiling entry function '_ZN5sb2001bEv' for 'sm_100a'
ptxas info    : Function properties for _ZN5sb2001bEv
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 40 registers, used 1 barriers, 264 bytes smem
"""
    rows = parse_ptxas_info(text)
    assert [r["kernel"] for r in rows] == ["_ZN5sb2001aEv", "_ZN5sb2001bEv"]
    assert (rows[0]["registers"], rows[0]["stack"], rows[0]["spill_stores"], rows[0]["spill_loads"], rows[0]["smem"]) == (168, 48, 44, 40, 1024)
    assert (rows[1]["registers"], rows[1]["smem"], rows[1]["spill_stores"]) == (40, 264, 0)


def test_gated_mlp_activations():
    """``--draft-hidden-act``: SiLU on the fused kernel path, GELU variants and ReLU element-wise, anything else refused by name."""
    import pytest
    import torch

    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.models.layers import MLP

    base = dict(model_type="llama", hidden_size=16, intermediate_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, vocab_size=10)
    acts = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu, "relu": torch.relu,
            "gelu_pytorch_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}
    x = torch.randn(5, 16)
    for name, fn in acts.items():
        mlp = MLP(TransformerLayerConfig(**base, hidden_act=name))
        gate, up = (x @ mlp.gate_up_proj.weight.t()).chunk(2, dim=-1)
        assert torch.allclose(mlp(x), (fn(gate) * up) @ mlp.down_proj.weight.t(), atol=1e-6)
    with pytest.raises(ValueError, match="not supported"):
        MLP(TransformerLayerConfig(**base, hidden_act="tanh"))
