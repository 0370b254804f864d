"""DFlash, DSpark and P-EAGLE on a GPU: the bf16 kernel path against the fp32 CPU model, at head
dims the attention kernels serve (64: ``mma.sync``; 128: tcgen05), and a few CUDA-graph steps."""

import copy
import tempfile

import pytest
import torch

from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.dflash import DFlashDraftModel
from speculators_b200.models.dspark import DSparkDraftModel
from speculators_b200.models.peagle import PEagleDraftModel
from speculators_b200.train import Trainer, TrainerConfig
from speculators_b200.train.synthetic import SyntheticLoader
from speculators_b200.verifier.model import write_random_verifier_stub

from conftest import make_tiny_batch

pytestmark = pytest.mark.gpu

VOCAB, DRAFT_VOCAB, HIDDEN = 512, 128, 128


def _verifier(tmp_path, head_dim):
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=HIDDEN, intermediate_size=256, num_hidden_layers=4,
               num_attention_heads=2, num_key_value_heads=1, head_dim=head_dim, vocab_size=VOCAB, max_position_embeddings=1024,
               rms_norm_eps=1e-6, rope_theta=10000.0, hidden_act="silu")
    return cfg, write_random_verifier_stub(str(tmp_path / f"verifier{head_dim}"), cfg, dtype=torch.float32)


def _maps():
    g = torch.Generator().manual_seed(1)
    t2d = torch.zeros(VOCAB, dtype=torch.bool)
    t2d[torch.randperm(VOCAB, generator=g)[:DRAFT_VOCAB]] = True
    kept = torch.nonzero(t2d).squeeze(1)
    return t2d, kept - torch.arange(DRAFT_VOCAB)


def _batch():
    b = make_tiny_batch(T=200, docs=(70, 90, 30), pad=10, hidden=HIDDEN, aux=3, vocab=VOCAB)
    b["position_ids"] = b["position_ids"] - 1
    return b


def _build(algo, tmp_path, head_dim):
    cfg, vdir = _verifier(tmp_path, head_dim)
    t2d, d2t = _maps()
    torch.manual_seed(0)
    common = dict(t2d=t2d, d2t=d2t, draft_vocab_size=DRAFT_VOCAB, verifier_name_or_path=vdir, target_layer_ids=[1, 2, 3], mask_token_id=5)
    if algo == "peagle":
        layer_cfg = TransformerLayerConfig(**dict(cfg, num_hidden_layers=1))
        model = PEagleDraftModel.from_training_args(layer_cfg, norm_before_residual=True, norm_before_fc=True, norm_output=True, **common)
        kwargs, _ = PEagleDraftModel.get_trainer_kwargs(loss_fn="kl_div", num_depths=4)
        return model, kwargs
    layer_cfg = TransformerLayerConfig(**dict(cfg, num_hidden_layers=2, sliding_window=64, layer_types=["full_attention", "sliding_attention"]))
    cls, extra = (DFlashDraftModel, {}) if algo == "dflash" else (DSparkDraftModel, {"markov_rank": 16, "markov_head_type": "gated"})
    model = cls.from_training_args(layer_cfg, block_size=8, **extra, **common)
    # every supervised position becomes an anchor, so CPU and GPU see the same blocks
    kwargs, _ = cls.get_trainer_kwargs(loss_fn="ce", max_anchors=256, per_position_loss_weight="dpace")
    return model, kwargs


@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("algo", ["dflash", "dspark", "peagle"])
def test_gpu_loss_matches_cpu_fp32(algo, head_dim, tmp_path):
    model, kwargs = _build(algo, tmp_path, head_dim)
    batch = _batch()
    torch.manual_seed(3)
    _, loss_cpu, _ = model(**batch, **kwargs)
    gpu = copy.deepcopy(model).to("cuda", torch.bfloat16)
    torch.manual_seed(3)
    _, loss_gpu, metrics = gpu(**{k: v.cuda() for k, v in batch.items()}, **kwargs)
    # P-EAGLE draws its deeper positions at random (different generators per device): looser bound
    rel = 0.35 if algo == "peagle" else 0.08
    assert abs(float(loss_gpu) - float(loss_cpu)) < rel * abs(float(loss_cpu)) + 0.05, (float(loss_gpu), float(loss_cpu))
    loss_gpu.backward()
    grads = [p.grad for p in gpu.parameters() if p.requires_grad and p.grad is not None]
    assert grads and all(torch.isfinite(g).all() for g in grads)
    assert all(torch.isfinite(v).all() for v in metrics.values() if torch.is_tensor(v))


@pytest.mark.parametrize("algo", ["dflash", "dspark", "peagle"])
def test_cuda_graph_steps(algo, tmp_path, monkeypatch):
    # P-EAGLE's step is graph-capturable only with the fixed-shape COD sampler (opt-in)
    monkeypatch.setenv("SB200_PEAGLE_FIXED_SHAPE", "1")
    model, kwargs = _build(algo, tmp_path, 128)
    batch = _batch()
    trainer = Trainer(model, TrainerConfig(lr=1e-3, num_epochs=1, save_path=tempfile.mkdtemp(), train_call_kwargs=kwargs, scheduler_type="none",
                                           log_freq=10**9, use_cuda_graph=True, device="cuda:0"), SyntheticLoader([batch], 6))
    losses = [float(trainer.train_step(batch)[0].item()) for _ in range(6)]
    assert all(torch.isfinite(torch.tensor(losses))), losses
    assert min(losses[3:]) < losses[0], losses
    assert trainer._graphed is not None and len(trainer._graphed.cache) == 1  # noqa: SLF001


# ------------------------------------------------------------------ MTP with a mixture-of-experts layer
def _moe_mtp(tmp_path, head_dim):
    from speculators_b200.config import SpeculatorsConfig, VerifierConfig
    from speculators_b200.models.mtp import MTPDraftModel
    from speculators_b200.models.mtp.config import MTPSpeculatorConfig
    from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

    heads = 512 // head_dim
    cfg = dict(architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next", hidden_size=512, intermediate_size=512, num_hidden_layers=2,
               num_attention_heads=heads, num_key_value_heads=max(1, heads // 2), head_dim=head_dim, vocab_size=VOCAB,
               max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=10000.0, partial_rotary_factor=0.25, hidden_act="silu",
               num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, shared_expert_intermediate_size=256, norm_topk_prob=True)
    vdir = write_random_verifier_stub(str(tmp_path / f"moe_verifier{head_dim}"), cfg, dtype=torch.float32)
    torch.manual_seed(0)
    model = MTPDraftModel(MTPSpeculatorConfig(
        transformer_layer_config=TransformerLayerConfig(**cfg),
        speculators_config=SpeculatorsConfig(algorithm="mtp", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=3)],
                                             default_proposal_method="greedy", verifier=VerifierConfig.from_pretrained(vdir)),
    ))
    model.load_verifier_weights()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.requires_grad and p.ndim >= 2:
                p.normal_(0.0, 0.05)
    kwargs, _ = MTPDraftModel.get_trainer_kwargs(num_speculative_steps=3, step_weight_beta=0.6)
    g = torch.Generator().manual_seed(3)
    T = 300
    hs = torch.randn(1, T, 512, generator=g)
    batch = dict(input_ids=torch.randint(0, VOCAB, (1, T), generator=g), hidden_states=hs / hs.pow(2).mean(-1, keepdim=True).sqrt(),
                 loss_mask=torch.rand(1, T, generator=g) > 0.3, position_ids=torch.arange(T).unsqueeze(0))
    return model, kwargs, batch


@pytest.mark.parametrize("head_dim", [64, 256])
def test_moe_mtp_gpu_loss_and_training_step(tmp_path, head_dim):
    """The MoE MTP head (gated attention, routed + shared experts on the grouped tcgen05 GEMM, head dim 256 on
    the attention kernels) in bf16 on the GPU against the fp32 CPU model, then optimizer steps through the trainer."""
    from speculators_b200 import ops

    model, kwargs, batch = _moe_mtp(tmp_path, head_dim)
    _, loss_cpu, _ = model(**batch, **kwargs)
    gpu = copy.deepcopy(model).to("cuda", torch.bfloat16)
    dev_batch = {k: (v.cuda().to(torch.bfloat16) if v.is_floating_point() else v.cuda()) for k, v in batch.items()}
    before = ops.native().launch_count()
    _, loss_gpu, _ = gpu(**dev_batch, **kwargs)
    loss_gpu.backward()
    torch.cuda.synchronize()
    ops.check_gemm_status()
    assert ops.native().launch_count() - before > 30
    assert abs(float(loss_gpu) - float(loss_cpu)) < 0.03 * abs(float(loss_cpu)) + 0.05, (float(loss_gpu), float(loss_cpu))
    assert all(torch.isfinite(p.grad).all() for p in gpu.parameters() if p.requires_grad and p.grad is not None)
    trainer = Trainer(copy.deepcopy(model), TrainerConfig(lr=2e-3, num_epochs=1, save_path=tempfile.mkdtemp(), train_call_kwargs=kwargs,
                                                          optimizer="adamw", scheduler_type="none", log_freq=10**9, device="cuda:0"),
                      SyntheticLoader([batch], 6))
    losses = [float(trainer.train_step(batch)[0]) for _ in range(6)]
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses
    assert trainer._graphed is not None and len(trainer._graphed.cache) == 1  # noqa: SLF001 - experts on one rank: the step is captured
    trainer.check_device_status()
