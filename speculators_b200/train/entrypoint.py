"""The training entry point behind ``scripts/train.py``.

``main(cfg)`` wires a resolved ``TrainConfig`` into a run: seeds, loggers,
process topology, vocabulary mappings, the draft model (from a checkpoint, a
decoder config file, or synthesised from the verifier config and the
decoder-shaping flags), data loaders over the selected hidden-state backend, the
``Trainer``.  Call structure and rules follow scripts/train.py:535-717 of the
reference; the helpers mirror :110-532 (``create_transformer_layer_config``,
``load_draft_transformer_layer_config``, ``parse_vocab_mappings``,
``build_draft_model``).
"""

from __future__ import annotations

import argparse
import copy
import gc
import logging
import os
import random
import warnings
from pathlib import Path

import numpy as np
import torch

from speculators_b200.hs_connectors import HiddenStatesBackend
from speculators_b200.layer_config import TransformerLayerConfig, read_config_json
from speculators_b200.model import SpeculatorModel
from speculators_b200.models.eagle3.data import shift_batch
from speculators_b200.models.mtp.data import shift_batch_mtp
from speculators_b200.models.utils import get_verifier_config, resolve_draft_intermediate_size
from speculators_b200.parallel.distributed import get_rank, is_distributed, maybe_destroy_distributed, maybe_setup_distributed
from speculators_b200.train.config import TrainConfig
from speculators_b200.train.dataloader import create_train_val_loaders
from speculators_b200.train.logger import log_run_config, setup_metric_logger, setup_root_logger
from speculators_b200.train.trainer import Trainer, TrainerConfig
from speculators_b200.train.utils import resolve_mask_token_id
from speculators_b200.train.vocab_mapping import build_vocab_mappings_from_distribution, get_target_vocab_size
from speculators_b200.utils.loading import is_config_only_dir

log = logging.getLogger("speculators")

DRAFT_ARCHS = ("llama", "qwen3")
_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}

__all__ = [
    "build_draft_model", "create_transformer_layer_config", "load_draft_transformer_layer_config", "main",
    "parse_vocab_mappings", "set_seed",
]


def set_seed(seed: int, deterministic: bool = False) -> None:
    random.seed(seed)
    np.random.seed(seed)  # noqa: NPY002
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False


def _apply_mrope_full_head_hack(rope: dict, head_dim: int, enabled: bool) -> None:
    """Multimodal verifiers rotate only part of each head (``partial_rotary_factor <
    1`` with ``mrope_section``); the draft rotates the full head, so the sections are
    scaled by the integer ``1 / factor``."""
    if "mrope_section" not in rope:
        return
    partial = float(rope.get("partial_rotary_factor", 1.0))
    if partial >= 1.0:
        return
    if not enabled:
        log.warning("mrope_full_head_hack=False with partial_rotary_factor=%s < 1.0 can cause trainer / vLLM partial-rotation mismatch.", partial)
        return
    inv = 1.0 / partial
    if abs(inv - round(inv)) > 1e-6:
        raise ValueError(f"mrope_full_head_hack cannot rescale mrope_section because 1/partial_rotary_factor={inv} is not an integer.")
    scaled = [int(x) * int(round(inv)) for x in rope["mrope_section"]]
    if 2 * sum(scaled) != head_dim:
        raise ValueError(f"mrope_full_head_hack rescaling produced inconsistent mrope_section {scaled}: 2*sum={2 * sum(scaled)} but head_dim={head_dim}.")
    log.warning("MRoPE full-head hack applied: partial_rotary_factor %s -> 1.0, mrope_section %s -> %s.", partial, rope["mrope_section"], scaled)
    rope["mrope_section"] = scaled
    rope["partial_rotary_factor"] = 1.0


def create_transformer_layer_config(verifier_name_or_path: str, num_layers: int, draft_arch: str, hidden_act: str | None, sliding_window: int,
                                    full_attention_indices: list[int], mrope_full_head_hack: bool = True, trust_remote_code: bool = False) -> TransformerLayerConfig:
    """Draft decoder config derived from the verifier's: same widths, vocabulary,
    norm epsilon and rotary settings; ``num_layers`` layers that use a sliding
    window unless listed in ``full_attention_indices``."""
    if draft_arch not in DRAFT_ARCHS:
        raise ValueError(f"Unknown draft architecture: {draft_arch}. Available: {list(DRAFT_ARCHS)}")
    v = get_verifier_config(verifier_name_or_path, trust_remote_code)
    act = hidden_act or v.get("hidden_act") or v.get("hidden_activation")
    if act is None:
        raise AttributeError("the verifier config has neither 'hidden_act' nor 'hidden_activation'")
    head_dim = v.get("head_dim") if "head_dim" in v else None
    nh, nkv = int(v.num_attention_heads), int(v.num_key_value_heads)
    if head_dim and v.hidden_size % nh != 0 and v.hidden_size % head_dim == 0:
        nh = v.hidden_size // head_dim
        if nh % nkv:
            nkv = nh
    resolved_head_dim = head_dim or v.hidden_size // nh
    if full_attention_indices and (min(full_attention_indices) < 0 or max(full_attention_indices) >= num_layers):
        raise ValueError("Full attention indices must be valid draft layer ids in range [0, num_layers).")
    layer_types = ["full_attention" if i in full_attention_indices else "sliding_attention" for i in range(num_layers)]
    cfg = {
        "model_type": draft_arch, "vocab_size": v.vocab_size, "hidden_size": v.hidden_size,
        "intermediate_size": resolve_draft_intermediate_size(v), "num_hidden_layers": num_layers, "num_attention_heads": nh,
        "num_key_value_heads": nkv, "hidden_act": act, "max_position_embeddings": v.max_position_embeddings,
        "initializer_range": v.get("initializer_range", 0.02), "rms_norm_eps": v.rms_norm_eps, "head_dim": resolved_head_dim,
        "tie_word_embeddings": False, "sliding_window": sliding_window, "use_sliding_window": "sliding_attention" in layer_types,
        "layer_types": layer_types, "rope_theta": float(v.rope_theta),
    }
    rope = v.get("rope_parameters") or v.get("rope_scaling")
    if isinstance(rope, dict):
        rope = copy.deepcopy(rope)
        if "rope_theta" not in rope and ("sliding_attention" in rope or "full_attention" in rope):
            rope = dict(rope.get("sliding_attention") or rope.get("full_attention") or {})
            rope.setdefault("rope_type", "default")
        rope.setdefault("rope_theta", float(v.rope_theta))
        _apply_mrope_full_head_hack(rope, resolved_head_dim, mrope_full_head_hack)
        rope.pop("type", None)
        rope.pop("mrope_interleaved", None)
        if "mrope_section" not in rope:
            rope.pop("partial_rotary_factor", None)
        cfg["rope_parameters"] = rope
        cfg["rope_theta"] = float(rope["rope_theta"])
    return TransformerLayerConfig(**cfg)


def load_draft_transformer_layer_config(draft_config: str, verifier_name_or_path: str, trust_remote_code: bool = False) -> TransformerLayerConfig:
    data = read_config_json(draft_config)
    if "transformer_layer_config" in data:  # a full speculator config: take its decoder part
        data = data["transformer_layer_config"]
    if not data.get("model_type"):
        raise ValueError(
            "--draft-config must define a 'model_type' (e.g. 'llama' for eagle3/peagle, 'qwen3' for dflash); none was "
            f"found in the config loaded from '{draft_config}'."
        )
    cfg = TransformerLayerConfig(**data)
    v = get_verifier_config(verifier_name_or_path, trust_remote_code)
    if cfg.hidden_size != v.hidden_size:
        raise ValueError(
            f"--draft-config hidden_size ({cfg.hidden_size}) must match the verifier hidden_size ({v.hidden_size}). "
            "Draft/verifier hidden-size mismatch is not yet supported."
        )
    if cfg.vocab_size != v.vocab_size:
        log.warning("Overriding --draft-config vocab_size (%s) with the verifier vocab_size (%s). Use --draft-vocab-size to control the pruned draft vocabulary.", cfg.vocab_size, v.vocab_size)
        cfg.vocab_size = v.vocab_size
    return cfg


def _load_mappings(d2t_path, t2d_path, expected: int | None):
    log.info("Loading vocab mappings from '%s' and '%s'", d2t_path, t2d_path)
    d2t = torch.from_numpy(np.load(d2t_path))
    t2d = torch.from_numpy(np.load(t2d_path))
    if expected and expected != d2t.shape[0]:
        raise ValueError(f"Explicit vocab mapping files don't match --draft-vocab-size {expected}: d2t.shape={tuple(d2t.shape)}.")
    return d2t, t2d, d2t.shape[0]


def parse_vocab_mappings(args: argparse.Namespace):
    """-> ``(d2t, t2d, draft_vocab_size)``.  Explicit ``.npy`` files; else files cached in
    the data directory; else built from ``token_freq.pt`` (and cached); else the full
    verifier vocabulary (no mapping)."""
    if args.d2t_path or args.t2d_path:
        if not (args.d2t_path and args.t2d_path):
            raise ValueError("Both t2d and d2t must be provided together, or both must be omitted.")
        return _load_mappings(args.d2t_path, args.t2d_path, args.draft_vocab_size)
    data_path = Path(args.data_path)
    if (data_path / "t2d.npy").exists() and (data_path / "d2t.npy").exists():
        return _load_mappings(data_path / "d2t.npy", data_path / "t2d.npy", args.draft_vocab_size)
    freq_path = Path(args.token_freq_path or data_path / "token_freq.pt")
    if freq_path.exists() and args.draft_vocab_size is not None:
        log.info("No vocab mappings provided. Regenerating from token frequencies")
        d2t, t2d = build_vocab_mappings_from_distribution(
            torch.load(freq_path, weights_only=True), args.draft_vocab_size, get_target_vocab_size(None, args.verifier_name_or_path)
        )
        if get_rank() == 0:
            data_path.mkdir(parents=True, exist_ok=True)
            np.save(data_path / "d2t.npy", d2t.numpy())
            np.save(data_path / "t2d.npy", t2d.numpy())
        return d2t, t2d, d2t.shape[0]
    log.warning("No vocab mappings found, and can't generate new ones because either token_freq_path='%s' doesn't exist or --draft-vocab-size is None. Using full verifier vocab", freq_path)
    return None, None, int(get_verifier_config(args.verifier_name_or_path).vocab_size)


def _build_from_config_only(model_class, path: str, t2d, d2t, verifier_name_or_path: str | None = None):
    config = model_class.config_class.from_pretrained(path)
    spec = getattr(config, "speculators_config", None)
    if verifier_name_or_path and spec is not None and not spec.verifier.name_or_path:
        spec.verifier.name_or_path = verifier_name_or_path
    model = model_class(config=config)
    if hasattr(model, "load_vocab_mappings"):
        model.load_vocab_mappings(t2d, d2t)
    if hasattr(model, "load_verifier_weights"):
        model.load_verifier_weights()
    return model


def build_draft_model(args: argparse.Namespace, model_class: type[SpeculatorModel], t2d, d2t, draft_vocab_size: int | None) -> SpeculatorModel:
    if args.from_pretrained:
        if is_config_only_dir(args.from_pretrained):
            log.info("--from-pretrained points to a config-only directory ('%s'); initializing fresh draft weights from the saved speculator config.", args.from_pretrained)
            return _build_from_config_only(model_class, args.from_pretrained, t2d, d2t, args.verifier_name_or_path)
        return model_class.from_pretrained(args.from_pretrained, t2d=t2d, d2t=d2t, verifier=args.verifier_name_or_path)
    if args.speculator_type == "mtp":
        layer_config = get_verifier_config(args.verifier_name_or_path, getattr(args, "trust_remote_code", False))
    else:
        if args.draft_config:
            layer_config = load_draft_transformer_layer_config(args.draft_config, args.verifier_name_or_path, args.trust_remote_code)
        else:
            if not args.full_attention_indices:
                log.info("All %d draft layers using sliding window attention (window=%d). To use full attention on specific layers, pass '--full-attention-indices <layer_ids>'.", args.num_layers, args.sliding_window)
            layer_config = create_transformer_layer_config(
                args.verifier_name_or_path, args.num_layers, args.draft_arch, args.draft_hidden_act, args.sliding_window,
                args.full_attention_indices, args.draft_mrope_full_head_hack, args.trust_remote_code,
            )
        if args.speculator_type in ("peagle", "dflash", "dspark"):
            args.mask_token_id = resolve_mask_token_id(args.verifier_name_or_path, layer_config.vocab_size, args.mask_token_id, trust_remote_code=args.trust_remote_code)
    args.draft_vocab_size = draft_vocab_size
    return model_class.from_training_args(verifier_config=layer_config, t2d=t2d, d2t=d2t, **vars(args))


def _trainer_config(args, model_class, dtype, **extra) -> TrainerConfig:
    train_kwargs, val_kwargs = model_class.get_trainer_kwargs(**vars(args))
    return TrainerConfig(
        num_epochs=args.epochs, save_path=args.save_path, lr=args.lr, resume_from_checkpoint=not args.no_resume_from_checkpoint,
        train_call_kwargs=train_kwargs, val_call_kwargs=val_kwargs, optimizer=args.optimizer, weight_decay=args.weight_decay,
        muon_lr=args.muon_lr, muon_momentum=args.muon_momentum, muon_weight_decay=args.muon_weight_decay,
        muon_ns_steps=args.muon_ns_steps, muon_adjust_lr_fn=args.muon_adjust_lr_fn, scheduler_type=args.scheduler_type,
        scheduler_warmup_steps=args.scheduler_warmup_steps, scheduler_warmup_ratio=args.scheduler_warmup_ratio,
        scheduler_total_steps=args.scheduler_total_steps, scheduler_num_cosine_cycles=args.scheduler_num_cosine_cycles,
        checkpoint_freq=args.checkpoint_freq, save_best=args.save_best, hidden_states_dtype=dtype, log_freq=args.log_freq,
        fsdp_shard=args.fsdp_shard, max_steps=args.max_steps, **extra,
    )


def _run_online(args, model, model_class, dtype) -> None:
    """``--online-verifier-gpus N``: no hidden-state files and no server.  The first N ranks load the verifier
    (tensor-parallel, each its slices of the checkpoint) and run the packed rows of the dataset in the order the
    multipack sampler gives the trainer ranks; the other ranks train on the states that arrive in their NVLink
    rings.  The reference reaches the same end with a vLLM server on part of the GPUs and ``--on-missing
    generate`` (scripts/launch_vllm.py, docs/user_guide/tutorials/train.md:165-170)."""
    import torch.distributed as dist

    from speculators_b200.train.noise_transforms import AddUniformNoise
    from speculators_b200.train.online import OnlineSplit
    from speculators_b200.train.online_data import OnlineBatchPlan

    if args.speculator_type not in ("eagle3", "peagle"):
        raise ValueError("--online-verifier-gpus supports the eagle3 and peagle speculator types (hidden states paired token by token)")
    if not is_distributed() or dist.get_world_size() <= args.online_verifier_gpus:
        raise ValueError("--online-verifier-gpus N needs a torchrun job of more than N ranks (N verifier ranks, the rest train)")
    if not torch.cuda.is_available():
        raise ValueError("--online-verifier-gpus needs CUDA devices with peer access (the hidden states travel over NVLink)")
    world, n_ver = dist.get_world_size(), int(args.online_verifier_gpus)
    # the trainer ranks are a sub-group of the job: their optimizer step uses the library collectives unless told otherwise
    # (the peer-memory step is exercised on whole jobs)
    os.environ.setdefault("SB200_COMM", "nccl")
    device = torch.device("cuda", torch.cuda.current_device())
    # seed 0: the multipack sampler's own default, i.e. the batches the file path forms for the same data and rank count
    plan = OnlineBatchPlan(args.data_path, args.total_seq_len, world - n_ver, seed=0, train_ratio=args.train_data_ratio)
    verifier_cfg = read_config_json(args.verifier_name_or_path)
    verifier_cfg = verifier_cfg.get("text_config", verifier_cfg)
    split = OnlineSplit(verifier_cfg, list(model.target_layer_ids), args.total_seq_len, device, n_verifier=n_ver, n_slots=args.online_ring_slots,
                        timeout_s=args.online_timeout, verifier_path=args.verifier_name_or_path, plan=plan,
                        transform=AddUniformNoise(std=args.noise_std) if args.noise_std > 0 else None)
    first_trainer = n_ver
    progress: list = [None, None]  # epoch and optimizer steps the trainer resumes from
    if split.topo.is_verifier:
        del model
        dist.broadcast_object_list(progress, src=first_trainer)
        budget = None if args.max_steps is None else max(0, int(args.max_steps) - int(progress[1])) + 1  # + the batch a trainer looks ahead
        served = split.serve(int(progress[0]), int(args.epochs), budget)
        log.info("in-job verifier served %d steps", served, extra={"override_rank0_filter": True})
    else:
        trainer = Trainer(model, _trainer_config(args, model_class, dtype, process_group=split.trainer_group), split.training_loader(), None)
        progress = [int(trainer.current_epoch), int(trainer.global_step)]
        dist.broadcast_object_list(progress, src=first_trainer)
        trainer.run_training()
        del trainer
    split.close()


def main(cfg: TrainConfig) -> None:
    args = argparse.Namespace(**cfg.flatten())
    set_seed(args.seed, args.deterministic_cuda)
    setup_root_logger()
    setup_metric_logger(loggers=args.logger, run_name=args.run_name, output_dir=args.log_dir)
    maybe_setup_distributed()
    log_run_config(cfg)
    if args.fsdp_shard and not is_distributed():
        raise ValueError("--fsdp-shard requires launching with torchrun/distributed training; otherwise parameters are not sharded.")
    if get_rank() == 0:
        cfg.save(args.save_path)
    dtype = _DTYPES.get(args.hidden_states_dtype) or getattr(torch, args.hidden_states_dtype)

    if args.speculator_type == "mtp":
        d2t = t2d = draft_vocab_size = None
        args.mask_token_id = None
    else:
        d2t, t2d, draft_vocab_size = parse_vocab_mappings(args)
    registry = SpeculatorModel.registry or {}
    if args.speculator_type not in registry:
        raise ValueError(f"Unknown speculator type: {args.speculator_type}. Available: {list(registry)}")
    model_class = registry[args.speculator_type]
    model = build_draft_model(args, model_class, t2d, d2t, draft_vocab_size)
    num_target_layers = len(model.target_layer_ids)
    if args.speculator_type == "mtp":
        args.num_speculative_steps = model.config.num_speculative_steps

    if args.dry_run:
        model.to(dtype)
        if get_rank() == 0:
            log.info("[dry-run] Saving initialized checkpoint (%s) to '%s'", dtype, args.save_path)
            model.save_pretrained(args.save_path)
            log.info("[dry-run] Done. Validate this checkpoint, then train with '--from-pretrained %s'.", args.save_path)
        maybe_destroy_distributed()
        return

    if args.online_verifier_gpus > 0:
        _run_online(args, model, model_class, dtype)
        maybe_destroy_distributed()
        return

    hidden_size = model.config.transformer_layer_config.hidden_size
    preprocess = {"eagle3": shift_batch, "peagle": shift_batch, "mtp": shift_batch_mtp}.get(args.speculator_type)
    transfer = HiddenStatesBackend.registry[args.hidden_states_backend].from_train_args(args, args.data_path)
    train_loader, val_loader = create_train_val_loaders(
        data_path=args.data_path, total_seq_len=args.total_seq_len, hidden_states_dtype=dtype, noise_std=args.noise_std,
        transfer=transfer, vllm_endpoint=args.vllm_endpoint, on_missing=args.on_missing, on_generate=args.on_generate,
        verifier_name_or_path=args.verifier_name_or_path, request_timeout=args.request_timeout, max_retries=args.max_retries,
        hidden_size=hidden_size, num_target_layers=num_target_layers, num_workers=args.num_workers,
        prefetch_factor=args.prefetch_factor, preprocess=preprocess, train_data_ratio=args.train_data_ratio,
    )
    trainer = Trainer(model, _trainer_config(args, model_class, dtype), train_loader, val_loader)
    trainer.run_training()
    del trainer, model
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    maybe_destroy_distributed()
