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
