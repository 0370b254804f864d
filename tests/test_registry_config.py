import json

import pytest

from speculators_b200 import (
    Eagle3SpeculatorConfig, GreedyTokenProposalConfig, SpeculatorModelConfig, SpeculatorsConfig,
    TokenProposalConfig, VerifierConfig,
)
from speculators_b200.utils import ClassRegistryMixin


def test_registry_register_and_duplicates():
    class Base(ClassRegistryMixin):
        pass

    @Base.register("a")
    class A(Base):
        pass

    @Base.register_decorator
    class B(Base):
        pass

    assert Base.registry == {"a": A, "B": B}
    assert Base.registered_classes() == (A, B)
    with pytest.raises(ValueError):
        Base.register("a")(A)
    with pytest.raises(ValueError):
        Base.register(3)
    with pytest.raises(TypeError):
        Base.register_decorator("not a class")

    class Other(ClassRegistryMixin):
        pass

    with pytest.raises(ValueError):
        Other.registered_classes()


def test_proposal_polymorphism():
    cfg = TokenProposalConfig.model_validate({"proposal_type": "greedy", "speculative_tokens": 4})
    assert isinstance(cfg, GreedyTokenProposalConfig) and cfg.speculative_tokens == 4
    with pytest.raises(ValueError):
        GreedyTokenProposalConfig(speculative_tokens=0)


def _spec_cfg(default="greedy"):
    return SpeculatorsConfig(
        algorithm="eagle3", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=3)],
        default_proposal_method=default, verifier=VerifierConfig(name_or_path="v", architectures=["LlamaForCausalLM"]),
    )


def test_default_proposal_must_be_listed():
    with pytest.raises(ValueError):
        _spec_cfg(default="tree")


def test_eagle3_config_round_trip(tmp_path):
    cfg = Eagle3SpeculatorConfig(
        transformer_layer_config={"model_type": "llama", "hidden_size": 64, "num_attention_heads": 4, "vocab_size": 128},
        draft_vocab_size=32, norm_before_residual=True, eagle_aux_hidden_state_layer_ids=[1, 2, 3], speculators_config=_spec_cfg(),
    )
    cfg.save_pretrained(tmp_path)
    raw = json.loads((tmp_path / "config.json").read_text())
    assert raw["speculators_model_type"] == "eagle3"
    assert raw["architectures"] == ["Eagle3Speculator"]
    assert raw["transformer_layer_config"]["model_type"] == "llama"
    assert raw["speculators_config"]["proposal_methods"][0]["speculative_tokens"] == 3
    loaded = SpeculatorModelConfig.from_pretrained(tmp_path)
    assert isinstance(loaded, Eagle3SpeculatorConfig)
    assert loaded.transformer_layer_config.hidden_size == 64
    assert loaded.to_dict() == cfg.to_dict()


def test_exclusive_norm_flags():
    with pytest.raises(ValueError):
        Eagle3SpeculatorConfig(norm_before_fc=True, fc_norm=True)


def test_from_dict_requires_discriminator():
    with pytest.raises(ValueError):
        SpeculatorModelConfig.from_dict({"draft_vocab_size": 3})
    with pytest.raises(ValueError):
        SpeculatorModelConfig.from_dict({"speculators_model_type": "nope"})


def test_optimizer_and_attention_compat_modules(tmp_path):
    import torch

    from speculators_b200.models.attention import AttnSpec, create_float_mask
    from speculators_b200.models.utils import conditional_torch_compile
    from speculators_b200.train import TrainerConfig
    from speculators_b200.train.optimizers import build_optimizers, split_named_params_for_muon

    model = torch.nn.Sequential(torch.nn.Linear(8, 16, bias=False), torch.nn.LayerNorm(16))
    (engine,) = build_optimizers(model, TrainerConfig(lr=1e-2, num_epochs=1, save_path=str(tmp_path), optimizer="adamw"), device="cpu")
    before = engine.flat_w.clone()
    model(torch.randn(4, 8)).pow(2).sum().backward()
    engine.step()
    assert not torch.equal(engine.flat_w, before)
    muon, adamw = split_named_params_for_muon(model)
    assert [n for n, _ in muon] == ["0.weight"] and len(adamw) == 2
    with pytest.raises(ValueError, match="Unsupported optimizer"):
        build_optimizers(model, TrainerConfig(lr=1e-2, num_epochs=1, save_path=str(tmp_path), optimizer="sgd"), device="cpu")
    spec = AttnSpec(lo=torch.tensor([0, 0, 2], dtype=torch.int32), hi=torch.tensor([1, 2, 2], dtype=torch.int32))
    m = create_float_mask(spec, 3)
    assert m[1].tolist() == [0.0, 0.0, float("-inf")] and torch.isinf(m[2]).all()

    @conditional_torch_compile
    def f(x):
        return x + 1

    assert f(1) == 2 and conditional_torch_compile(dynamic=True)(f)(2) == 3


def test_eagle_converter_helpers_and_legacy_model_name(tiny_verifier_dir, tiny_vocab_maps, tmp_path):
    import torch

    from speculators_b200.convert.eagle.eagle3_legacy_model import Eagle3Speculator
    from speculators_b200.convert.eagle.utils import (
        build_llama_config_dtype_kwarg, build_llama_config_rope_kwargs, detect_fusion_bias_and_layernorms, find_vocab_size,
    )
    from tests.conftest import make_tiny_eagle3

    assert detect_fusion_bias_and_layernorms({"fc.bias": torch.zeros(1), "post_embedding_layernorm.weight": torch.zeros(1)}) == (True, True)
    assert detect_fusion_bias_and_layernorms({"fc.weight": torch.zeros(1)}) == (False, False)
    assert find_vocab_size({"a": {"b": {"vocab_size": 7}}}) == 7 and find_vocab_size({"a": 1}) is None
    assert build_llama_config_dtype_kwarg(None) == {} and build_llama_config_dtype_kwarg("bfloat16") == {"torch_dtype": "bfloat16"}
    rope = build_llama_config_rope_kwargs(5e5, {"type": "llama3", "factor": 8.0})
    assert rope["rope_parameters"] == {"rope_theta": 5e5, "rope_type": "llama3", "factor": 8.0} and rope["rope_scaling"]["factor"] == 8.0
    assert build_llama_config_rope_kwargs()["rope_parameters"] == {"rope_theta": 10000.0, "rope_type": "default"}

    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    model.save_pretrained(tmp_path / "ckpt")
    legacy = Eagle3Speculator.from_pretrained(str(tmp_path / "ckpt"), verifier=tiny_verifier_dir, verifier_attachment_mode="detached")
    assert torch.equal(legacy.fc.weight, model.fc.weight)
    built = Eagle3Speculator(model.config, verifier=None, verifier_attachment_mode="detached", reduce_vocab_size=False, has_drafter_embedding=False)
    assert built.d2t is None and not built.embed_tokens.weight.requires_grad
    with pytest.raises(ValueError, match="detached"):
        Eagle3Speculator(model.config, verifier_attachment_mode="full")


def test_reference_module_paths_and_names_resolve():
    """Names a user of the reference imports from its module paths exist here under the same
    paths (aliases over this package's own implementations where the design differs)."""
    import importlib

    expected = {
        "speculators_b200.models": ["Eagle3DraftModel", "DFlashSpeculatorConfig", "MTPDraftModel", "PEagleDraftModel", "DSparkDraftModel"],
        "speculators_b200.models.eagle3": ["shift_batch"],
        "speculators_b200.models.mtp": ["shift_batch_mtp"],
        "speculators_b200.models.eagle3.model_definitions": ["Eagle3FirstLayerMixin", "LlamaDecoderEagle3FirstLayer", "Qwen3DecoderEagle3FirstLayer", "model_classes"],
        "speculators_b200.models.dflash.model_definitions": ["Qwen3DFlashAttention", "Qwen3DFlashDecoderLayer", "apply_rotary_pos_emb"],
        "speculators_b200.models.mtp.model_definitions": ["MTPLayerMixin", "mtp_model_classes", "resolve_model_type"],
        "speculators_b200.models.attention": ["ALL_ATTENTION_FUNCTIONS"],
        "speculators_b200.models.utils": ["DEFAULT_TARGET_LAYER_IDS_WARNING", "flatten_rope_parameters", "resolve_draft_intermediate_size"],
        "speculators_b200.train.distributed": ["apply_fully_sharded", "get_dp_group", "get_sp_rank", "maybe_setup_distributed"],
        "speculators_b200.train.graceful_shutdown": ["DEFAULT_SHUTDOWN_TIMEOUT", "TrainingInterruptedError"],
        "speculators_b200.train.logger": ["TB_SUPPORTED_TYPES", "IsRank0Filter"],
        "speculators_b200.convert": ["convert_model"],
        "speculators_b200.convert.eagle": ["Eagle3Converter"],
        "speculators_b200.convert.dflash": ["DFlashConverter"],
        "speculators_b200.convert.mtp": ["MTPConverter", "MTP_EXACT_REMAP", "MTP_PREFIX_REMAP"],
        "speculators_b200.convert.utils": ["download_checkpoint_from_hub", "ensure_checkpoint_is_local"],
        "speculators_b200.data_generation.vllm_client": ["wait_for_lock", "wait_for_lock_async"],
        "speculators_b200.utils.util": ["is_npu_available"],
        "speculators_b200.__main__": ["app", "main"],
    }
    for module, names in expected.items():
        mod = importlib.import_module(module)
        for name in names:
            assert hasattr(mod, name), f"{module}.{name}"
    from speculators_b200.models.mtp.model_definitions import mtp_model_classes

    assert {"qwen3", "qwen3_next"} <= set(mtp_model_classes) and mtp_model_classes["qwen3"].first_layer_class.__name__ == "MTPLayer"
    from speculators_b200.models.dflash.model_definitions import apply_rotary_pos_emb
    import torch

    q, k = torch.randn(1, 2, 3, 8), torch.randn(1, 2, 5, 8)
    cos, sin = torch.ones(1, 5, 8), torch.zeros(1, 5, 8)
    rq, rk = apply_rotary_pos_emb(q, k, cos, sin)
    assert torch.equal(rq, q) and torch.equal(rk, k)  # identity rotation
