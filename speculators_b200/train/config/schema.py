"""Typed training configuration: the single source of truth for every flag.

Each tunable is one pydantic field inside a thematic group; the ``train.py`` CLI
is generated from these fields (``resolution.py``) and the YAML file format mirrors
the nesting.  Field names, defaults and derived defaults are those of the
reference (src/speculators/train/config/schema.py:58-531, 609-703) so existing
command lines and ``run.yaml`` files keep working:

* precedence is ``flag > yaml > default``;
* per-algorithm defaults: eagle3 -> ``draft_arch=llama``, ``norm_before_fc =
  norm_output = True``; dflash -> 5 layers, block size 16, CE loss, D-PACE
  weights; everything else -> ``qwen3``, 1 layer, block size 8, KL loss;
  ``muon_lr = 10 * lr``;
* D-PACE requires CE and ``0 < dpace_alpha <= 1``.

Unlike the reference this is a plain ``BaseModel`` tree: the layering is an
explicit deep merge done by ``resolution.build_from_sources`` rather than
pydantic-settings source ordering.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from types import MappingProxyType
from typing import Any, Literal

from pydantic import BaseModel, ConfigDict, Field, PrivateAttr, field_validator, model_validator

from speculators_b200.losses import resolve_loss_config

DEFAULT_REQUEST_TIMEOUT = 120.0
DEFAULT_MAX_RETRIES = 3

# field markers understood by the CLI generator
CLI_BOOL_OPTIONAL: dict[str, Any] = {"cli_bool": "optional"}  # render a False-default bool as --x/--no-x
CLI_REQUIRED: dict[str, Any] = {"cli_required": True}  # must come from a flag or the YAML file
CLI_CHOICES_BACKENDS: dict[str, Any] = {"cli_choices": "hidden_states_backends"}

__all__ = ["CONFIG_DESTS", "GROUPS", "ROOT_FIELDS", "TrainConfig", "nest_flat"]


class _Group(BaseModel):
    model_config = ConfigDict(extra="ignore", validate_assignment=False)


class VerifierArgs(_Group):
    verifier_name_or_path: str = Field(default="", json_schema_extra=CLI_REQUIRED, description="Verifier model: local path or hub id.")
    trust_remote_code: bool = Field(default=False, description="Allow custom code from the verifier repository.")


class DraftArgs(_Group):
    from_pretrained: str = Field(default="", description="Start from a complete speculators checkpoint (or a config-only directory).")
    draft_config: str = Field(default="", description="Decoder config (json file / directory) for the draft layers.")
    num_layers: int | None = Field(default=None, description="Number of draft decoder layers (default: 5 for dflash, else 1).")
    draft_arch: Literal["llama", "qwen3"] | None = Field(default=None, description="Draft decoder family (default: llama for eagle3, else qwen3).")
    draft_hidden_act: str = Field(default="silu", description="Draft MLP activation.")
    draft_mrope_full_head_hack: bool = Field(default=True, description="Expand MRoPE sections to the full head for multimodal verifiers.")
    target_layer_ids: list[int] | None = Field(default=None, description="Verifier layers whose hidden states feed the draft.")
    token_freq_path: str | None = Field(default=None, description="token_freq.pt used to build the draft vocabulary.")
    draft_vocab_size: int | None = Field(default=None, description="Draft vocabulary size (default: full verifier vocabulary).")
    d2t_path: str | None = Field(default=None, description="Explicit d2t.npy.")
    t2d_path: str | None = Field(default=None, description="Explicit t2d.npy.")
    mask_token_id: int | None = Field(default=None, description="Mask token id; resolved from the tokenizer when unset.")
    norm_before_residual: bool = Field(default=True, description="Normalise the hidden half before it becomes the residual.")
    embed_requires_grad: bool = Field(default=False, json_schema_extra=CLI_BOOL_OPTIONAL, description="Train the token embeddings.")
    norm_before_fc: bool | None = Field(default=None, description="One RMSNorm over the concatenated aux states before fc (default: True for eagle3).")
    fc_norm: bool = Field(default=False, description="One RMSNorm per aux state before concatenation.")
    norm_output: bool | None = Field(default=None, description="Feed post-norm hidden states to the next TTT step (default: True for eagle3).")
    sliding_window: int = Field(default=2048, description="Window of sliding-attention draft layers.")
    full_attention_indices: list[int] = Field(default_factory=list, description="Draft layers that use full attention instead of the window.")
    sliding_window_non_causal: bool = Field(default=False, description="DFlash: sliding layers attend bidirectionally inside a block.")
    draft_attn_impl: Literal["simple_flex_attention", "sdpa", "eager"] = Field(
        default="simple_flex_attention",
        description="Kept for command-line compatibility; attention always runs the package's own kernels (dense oracle on CPU).",
    )


class DataArgs(_Group):
    data_path: str = Field(default="./output", description="Directory of the preprocessed dataset.")
    hidden_states_backend: str = Field(default="file", json_schema_extra=CLI_CHOICES_BACKENDS, description="Hidden-state transport.")
    total_seq_len: int = Field(default=8192, description="Packed tokens per batch (per rank).")
    train_data_ratio: float = Field(default=0.9, description="Fraction of samples used for training (rest: validation).")
    noise_std: float = Field(default=0.05, description="Std of the uniform noise added to hidden states during training.")
    hidden_states_dtype: str = Field(default="bfloat16", description="dtype hidden states are cast to (and the compute dtype).")
    num_workers: int = Field(default=12, description="DataLoader workers.")
    prefetch_factor: int = Field(default=4, description="Batches prefetched per worker.")
    max_anchors: int = Field(default=512, description="Anchors per batch (DFlash / DSpark / P-EAGLE).")

    @field_validator("hidden_states_dtype")
    @classmethod
    def _names_a_supported_dtype(cls, v: str) -> str:
        import torch  # only needed to check the name; keeps the schema importable without it otherwise

        resolved = getattr(torch, v, None)
        if not isinstance(resolved, torch.dtype):  # torch.nn, torch.cuda, ... exist but are not dtypes
            raise ValueError("hidden_states_dtype must name a torch dtype, e.g. `bfloat16`.")
        if resolved is torch.float16:
            raise ValueError("hidden_states_dtype float16 is not supported (it needs gradient scaling); use bfloat16.")
        return v


class GenerationArgs(_Group):
    vllm_endpoint: str = Field(default="http://localhost:8000/v1", description="OpenAI-compatible endpoint of the verifier server.")
    on_missing: Literal["generate", "skip", "warn", "raise"] = Field(default="generate", description="What to do when a sample has no cached hidden states.")
    on_generate: Literal["cache", "delete"] = Field(default="delete", description="Keep or drop hidden states generated on the fly.")
    request_timeout: float = Field(default=DEFAULT_REQUEST_TIMEOUT, description="Seconds per generation request.")
    max_retries: int = Field(default=DEFAULT_MAX_RETRIES, description="Retries per generation request.")
    online_verifier_gpus: int = Field(default=0, description="Run the verifier inside the job, tensor-parallel on the first N ranks; the other ranks train on hidden states handed GPU to GPU (0: off).")
    online_ring_slots: int = Field(default=4, description="Samples the in-job verifier may run ahead of a trainer rank.")
    online_timeout: float = Field(default=600.0, description="Seconds a rank of the in-job verifier / trainer split waits for the other side.")


class LossArgs(_Group):
    loss_implementation: Literal["fused", "eager"] = Field(default="fused", description="Fused kernels or dense PyTorch losses.")
    loss_fn: str | None = Field(default=None, description="Loss name or JSON dict of weights (default: ce for dflash, else kl_div).")
    ttt_steps: int = Field(default=3, description="EAGLE-3 training-time-test passes.")
    ttt_step_loss_decay: float = Field(default=1.0, description="Loss weight decay**step.")

    @field_validator("loss_fn")
    @classmethod
    def _known_loss(cls, value: str | None) -> str | None:
        if value is not None:
            resolve_loss_config(value, "eager")
        return value


class OptimizerArgs(_Group):
    optimizer: Literal["adamw", "muon"] = Field(default="muon", description="adamw, or muon for 2-D weights + adamw for the rest.")
    lr: float = Field(default=1e-4, description="AdamW learning rate.")
    weight_decay: float = Field(default=0.01, description="AdamW weight decay.")
    muon_lr: float | None = Field(default=None, description="Muon learning rate (default: 10 * lr).")
    muon_momentum: float = Field(default=0.95, description="Muon momentum (Nesterov).")
    muon_weight_decay: float = Field(default=0.1, description="Decoupled weight decay of the Muon group.")
    muon_ns_steps: int = Field(default=5, description="Newton-Schulz iterations.")
    muon_adjust_lr_fn: Literal["original", "match_rms_adamw"] = Field(default="match_rms_adamw", description="How the Muon step is scaled with the matrix shape.")


class SchedulerArgs(_Group):
    scheduler_type: Literal["linear", "cosine", "none"] = Field(default="linear", description="Learning-rate schedule after warm-up.")
    scheduler_warmup_steps: int | None = Field(default=None, description="Linear warm-up steps (wins over the ratio).")
    scheduler_warmup_ratio: float | None = Field(default=None, description="Warm-up as a fraction of the total steps, in [0, 1].")
    scheduler_total_steps: int | None = Field(default=None, description="Steps the schedule spans (default: epochs * batches per epoch).")
    scheduler_num_cosine_cycles: float = Field(default=0.5, description="Cosine periods over the schedule (0.5: one descent to zero).")


class TrainerArgs(_Group):
    epochs: int = Field(default=20, description="Passes over the training split.")
    checkpoint_freq: float = Field(default=1.0, description=">= 1: every N epochs; < 1: fraction of an epoch.")
    save_best: bool = Field(default=False, description="Keep only the best validation epoch.")
    no_resume_from_checkpoint: bool = Field(default=False, description="Ignore existing checkpoints in --save-path.")
    log_freq: int = Field(default=1, description="Log metrics every N steps.")
    save_path: str = Field(default="./output/checkpoints", description="Checkpoint directory (also where a run resumes from).")
    fsdp_shard: bool = Field(default=False, description="Shard optimizer state and master weights across ranks.")
    max_steps: int | None = Field(default=None, gt=0, description="Stop after this many optimizer steps (a positive integer); default: run all epochs.")

    @field_validator("checkpoint_freq")
    @classmethod
    def _whole_epochs_or_a_fraction(cls, v: float) -> float:
        if v <= 0:
            raise ValueError("--checkpoint-freq must be > 0")
        if v > 1 and not float(v).is_integer():
            raise ValueError(f"--checkpoint-freq={v} is not an integer. Values > 1 are epoch counts and must be whole numbers.")
        return v


class LoggingArgs(_Group):
    logger: str = Field(default="", description="Comma-separated metric backends: tensorboard, wandb, trackio, mlflow.")
    log_dir: str = Field(default="./logs", description="Directory of the metric backends' files.")
    run_name: str | None = Field(default=None, description="Run name; {time}, {utc_time}, {rank}, {local_rank} are substituted.")


class DFlashArgs(_Group):
    block_size: int | None = Field(default=None, description="Draft block size (default: 16 for dflash, else 8).")
    sample_from_anchor: bool | None = Field(default=None, description="Slot 0 predicts (default: True for dspark).")
    dflash_decay_gamma: float = Field(default=4.0)
    per_position_loss_weight: Literal["fixed-exp-decay", "dpace"] | None = Field(default=None)
    dpace_alpha: float = Field(default=0.5)


class DSparkArgs(_Group):
    markov_rank: int = Field(default=256)
    markov_head_type: Literal["vanilla", "gated", "rnn"] = Field(default="vanilla")
    enable_confidence_head: bool = Field(default=True)
    confidence_head_with_markov: bool = Field(default=True)
    confidence_head_alpha: float = Field(default=1.0)


class PEagleArgs(_Group):
    num_depths: int = Field(default=8)
    down_sample_ratio: float = Field(default=0.7)
    down_sample_ratio_min: float = Field(default=0.2)


class MTPArgs(_Group):
    num_speculative_steps: int = Field(default=3)
    step_weight_beta: float = Field(default=0.6)


GROUPS: dict[str, type[_Group]] = {
    "verifier": VerifierArgs, "draft": DraftArgs, "data": DataArgs, "generation": GenerationArgs, "loss": LossArgs,
    "optimizer": OptimizerArgs, "scheduler": SchedulerArgs, "trainer": TrainerArgs, "logging": LoggingArgs,
    "dflash": DFlashArgs, "dspark": DSparkArgs, "peagle": PEagleArgs, "mtp": MTPArgs,
}


class TrainConfig(BaseModel):
    model_config = ConfigDict(extra="ignore", validate_assignment=False)

    _provenance: dict[str, str] = PrivateAttr(default_factory=dict)
    _argv: list[str] = PrivateAttr(default_factory=list)
    _backend_args: dict[str, Any] = PrivateAttr(default_factory=dict)

    speculator_type: str = Field(default="eagle3", description="eagle3, dflash, dspark, peagle or mtp.")
    dry_run: bool = Field(default=False, description="Build the draft, save it to --save-path and exit before training.")
    seed: int = Field(default=42, description="Seed of Python, NumPy and torch generators.")
    deterministic_cuda: bool = Field(default=False, description="Ask torch for deterministic algorithms (slower).")

    verifier: VerifierArgs = Field(default_factory=VerifierArgs)
    draft: DraftArgs = Field(default_factory=DraftArgs)
    data: DataArgs = Field(default_factory=DataArgs)
    generation: GenerationArgs = Field(default_factory=GenerationArgs)
    loss: LossArgs = Field(default_factory=LossArgs)
    optimizer: OptimizerArgs = Field(default_factory=OptimizerArgs)
    scheduler: SchedulerArgs = Field(default_factory=SchedulerArgs)
    trainer: TrainerArgs = Field(default_factory=TrainerArgs)
    logging: LoggingArgs = Field(default_factory=LoggingArgs)
    dflash: DFlashArgs = Field(default_factory=DFlashArgs)
    dspark: DSparkArgs = Field(default_factory=DSparkArgs)
    peagle: PEagleArgs = Field(default_factory=PEagleArgs)
    mtp: MTPArgs = Field(default_factory=MTPArgs)

    # ---- bookkeeping (never serialised) -----------------------------------------
    @property
    def provenance(self) -> Mapping[str, str]:
        """Winning layer per flat field: ``flag`` | ``yaml`` | ``default``."""
        return MappingProxyType(self._provenance)

    @property
    def argv(self) -> Sequence[str]:
        return tuple(self._argv)

    @property
    def backend_args(self) -> Mapping[str, Any]:
        return MappingProxyType(self._backend_args)

    # ---- validators -----------------------------------------------------------------
    @model_validator(mode="after")
    def _resolve_derived_defaults(self) -> "TrainConfig":
        eagle3 = self.speculator_type == "eagle3"
        dflash = self.speculator_type == "dflash"
        if self.draft.draft_arch is None:
            self.draft.draft_arch = "llama" if eagle3 else "qwen3"
        if self.draft.norm_before_fc is None:
            self.draft.norm_before_fc = eagle3
        if self.draft.norm_output is None:
            self.draft.norm_output = eagle3
        if self.optimizer.muon_lr is None:
            self.optimizer.muon_lr = 10 * self.optimizer.lr
        if self.draft.num_layers is None:
            self.draft.num_layers = 5 if dflash else 1
        if self.dflash.per_position_loss_weight is None:
            self.dflash.per_position_loss_weight = "dpace" if dflash else "fixed-exp-decay"
        if self.loss.loss_fn is None:
            self.loss.loss_fn = "ce" if dflash else "kl_div"
        if self.dflash.block_size is None:
            self.dflash.block_size = 16 if dflash else 8
        return self

    @model_validator(mode="after")
    def _validate_dpace(self) -> "TrainConfig":
        if self.dflash.per_position_loss_weight == "dpace":
            if self.loss.loss_fn != "ce":
                raise ValueError("--per-position-loss-weight=dpace requires --loss-fn=ce")
            if not 0.0 < self.dflash.dpace_alpha <= 1.0:
                raise ValueError(f"--dpace-alpha must be in (0, 1], got {self.dflash.dpace_alpha}")
        return self

    # ---- flat view --------------------------------------------------------------------
    def flatten(self) -> dict[str, Any]:
        """Flat ``vars(args)``-shaped dict (schema order) consumed by the model
        classes' ``from_training_args`` / ``get_trainer_kwargs``."""
        out = {name: getattr(self, name) for name in ROOT_FIELDS}
        for gname, gmodel in GROUPS.items():
            group = getattr(self, gname)
            for fname in gmodel.model_fields:
                out[fname] = getattr(group, fname)
        out.update(self._backend_args)
        return out

    @classmethod
    def from_flat(cls, flat: dict[str, Any]) -> "TrainConfig":
        from speculators_b200.train.config.resolution import BACKEND_DESTS

        cfg = cls(**nest_flat({k: v for k, v in flat.items() if k in CONFIG_DESTS}))
        cfg._backend_args = {k: v for k, v in flat.items() if k in BACKEND_DESTS}
        return cfg

    @classmethod
    def from_sources(cls, *, cli: dict[str, Any], config_path: str | None = None, argv: list[str], backend_cli: dict[str, Any] | None = None) -> "TrainConfig":
        from speculators_b200.train.config import resolution

        return resolution.build_from_sources(cls, cli=cli, config_path=config_path, argv=argv, backend_cli=backend_cli)

    @classmethod
    def resolve(cls, argv: list[str] | None = None) -> "TrainConfig":
        from speculators_b200.train.config import resolution

        return resolution.resolve(cls, argv)

    def dump_yaml(self) -> str:
        from speculators_b200.train.config import artifacts

        return artifacts.dump_yaml(self)

    def save(self, save_dir: str) -> None:
        from speculators_b200.train.config import artifacts

        artifacts.save(self, save_dir)


ROOT_FIELDS: tuple[str, ...] = tuple(n for n in TrainConfig.model_fields if n not in GROUPS)


def _dest_to_group() -> dict[str, str | None]:
    mapping: dict[str, str | None] = dict.fromkeys(ROOT_FIELDS)
    for gname, gmodel in GROUPS.items():
        for fname in gmodel.model_fields:
            if fname in mapping:
                raise RuntimeError(f"duplicate config field '{fname}' across groups")
            mapping[fname] = gname
    return mapping


DEST_TO_GROUP: dict[str, str | None] = _dest_to_group()
CONFIG_DESTS: frozenset[str] = frozenset(DEST_TO_GROUP)


def nest_flat(flat: dict[str, Any]) -> dict[str, Any]:
    nested: dict[str, Any] = {}
    for dest, value in flat.items():
        group = DEST_TO_GROUP.get(dest)
        if group is None:
            nested[dest] = value
        else:
            nested.setdefault(group, {})[dest] = value
    return nested
