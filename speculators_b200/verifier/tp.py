"""Tensor-parallel verifier forward.

The reference runs its verifier in a vLLM server with ``--tensor-parallel-size``
(scripts/launch_vllm.py:104-163); a 70B-class verifier does not fit one GPU's worth of
throughput next to the trainer.  This is the in-framework counterpart of that server for dense
Llama / Qwen3 verifiers: the ranks of a process group split every layer Megatron-style

* q | k | v and gate | up column-parallel (each rank holds ``heads / R`` query heads, ``kv_heads / R``
  KV heads and ``intermediate / R`` MLP columns),
* o and down row-parallel: every rank multiplies its slice and the partial sums are all-reduced,

so a layer costs two all-reduces of ``[T, H]``.  On CUDA devices with peer access these are not
library calls: the row-parallel GEMM's epilogue stores its tiles into the owning rank's staging
area over NVLink and a second kernel reduces, adds the residual stream and writes every rank's
copy (``parallel/tp_comm.py``; ``SB200_TP_COMM=nccl`` keeps the NCCL all-reduce, the twin the
result is tested against).  All products run on the package's GEMM and
attention kernels through the same ``DecoderLayer`` the draft models use (built for the local
head / column counts).  Weights are the rank's slices of exactly the tensors ``RandomVerifier``
generates for a seed, so the result equals the single-device forward (tested with two gloo ranks).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.distributed as dist

from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.eagle3.attention import causal_document_interval
from speculators_b200.models.layers import DecoderLayer, RotaryTable
from speculators_b200.ops import AttnSpec
from speculators_b200.verifier.model import _seeded

__all__ = ["TensorParallelVerifier"]


class _ShardedCheckpoint:
    """Slices of the tensors of a Hugging Face safetensors checkpoint (single file or sharded with an
    index): a rank reads only the rows / columns it owns."""

    def __init__(self, path: str | Path):
        from speculators_b200.utils.loading import _weight_map, resolve_checkpoint_file

        self.path = Path(path)
        self.files = _weight_map(self.path)  # tensor name -> file
        self._resolve = resolve_checkpoint_file
        self._open: dict[str, object] = {}

    def _handle(self, key: str):
        from safetensors import safe_open

        file = self.files[key]
        if file not in self._open:
            self._open[file] = safe_open(str(self._resolve(self.path, file)), framework="pt", device="cpu")
        return self._open[file]

    def key(self, name: str) -> str | None:
        """The checkpoint's spelling of ``name`` (exact, or with a prefix such as ``language_model.``)."""
        if name in self.files:
            return name
        hits = [k for k in self.files if k.endswith("." + name) or k.endswith(name)]
        return min(hits, key=len) if hits else None

    def read(self, key: str, rows: tuple[int, int] | None = None, cols: tuple[int, int] | None = None) -> torch.Tensor:
        view = self._handle(key).get_slice(key)
        if rows is not None:
            return view[rows[0] : rows[1]]
        if cols is not None:
            return view[:, cols[0] : cols[1]]
        return view[:]

    def close(self) -> None:
        self._open.clear()


class TensorParallelVerifier:
    def __init__(self, config: TransformerLayerConfig | dict, group=None, seed: int = 0, device="cpu", dtype=torch.float32,
                 resident: bool = False, sliced_init: bool = False, max_tokens: int | None = None, comm: str | None = None):
        """``resident``: keep every layer's slices on the device after the first forward (a 70B-class
        verifier over 4 GPUs holds 35 GB per GPU) instead of regenerating them per call.
        ``sliced_init``: draw each rank's slices directly from a seed of their own instead of
        slicing the full tensors (``world`` times less work at start-up; the weights then differ
        from ``RandomVerifier``'s for the same seed, which only matters to tests)."""
        self.resident, self.sliced_init = bool(resident), bool(sliced_init)
        self._layers: dict[int, DecoderLayer] = {}
        self._checkpoint: _ShardedCheckpoint | None = None  # set by ``from_pretrained``: weights come from files, not from seeds
        # what a layer id names: False = the output of decoder layer ``id`` (``RandomVerifier``'s numbering); True = the
        # state after ``id`` layers, i.e. Hugging Face ``hidden_states[id]`` and the numbering of vLLM's
        # ``eagle_aux_hidden_state_layer_ids`` (0 = embeddings, ``num_hidden_layers`` = the last layer's output)
        self.layers_counted = False
        self.cfg = TransformerLayerConfig.from_any(config)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        c, R = self.cfg, self.world
        if R > 1 and (bool(c.attention_bias) or bool(c.mlp_bias)):
            # the bias of a row-parallel projection (o_proj, down_proj) would be added once per rank by the sum over the ranks
            raise ValueError("the tensor-parallel verifier does not support attention_bias / mlp_bias")
        if c.num_attention_heads % R or c.num_key_value_heads % R or c.intermediate_size % R:
            raise ValueError(f"heads ({c.num_attention_heads} / {c.num_key_value_heads}) and intermediate size ({c.intermediate_size}) "
                             f"must be divisible by the tensor-parallel size ({R})")
        self.seed, self.device, self.dtype = seed, torch.device(device), dtype
        self.rotary = RotaryTable(self.cfg).to(self.device)
        self.local_cfg = TransformerLayerConfig(**{
            **self.cfg.to_dict(), "num_attention_heads": c.num_attention_heads // R, "num_key_value_heads": c.num_key_value_heads // R,
            "intermediate_size": c.intermediate_size // R, "head_dim": c.head_dim,
        })
        with torch.device("meta"):  # names, shapes and order of a full layer's tensors (what the seeds are tied to)
            self._full_shapes = [(n, tuple(p.shape)) for n, p in DecoderLayer(self.cfg, 0).named_parameters()]
        self.comm = self._make_comm(comm, max_tokens)

    def _make_comm(self, choice: str | None, max_tokens: int | None):
        """The fused row-parallel exchange, or ``None`` for the library all-reduce.  Every rank of the
        group takes the same branch (the inputs of the decision are the same everywhere)."""
        import os

        from speculators_b200.parallel.tp_comm import TpComm

        choice = choice or os.environ.get("SB200_TP_COMM") or "auto"
        if choice not in ("auto", "peer", "nccl"):
            raise ValueError(f"comm must be 'peer', 'nccl' or None, got {choice!r}")
        able = (self.world > 1 and self.device.type == "cuda" and self.dtype == torch.bfloat16 and max_tokens is not None
                and TpComm.supported(int(self.cfg.hidden_size), self.world))
        if choice == "nccl" or (choice == "auto" and not able):
            return None
        if not able:
            raise ValueError("comm='peer' needs a CUDA device, bf16 weights, max_tokens and hidden_size / world a multiple of 256")
        comm = TpComm(self.group, int(max_tokens), int(self.cfg.hidden_size), self.device)
        comm.connect()
        return comm

    @classmethod
    def from_pretrained(cls, path: str | Path, group=None, device="cuda", dtype=torch.bfloat16, max_tokens: int | None = None,
                        comm: str | None = None) -> "TensorParallelVerifier":
        """A verifier with the weights of a Hugging Face checkpoint directory (``config.json`` + safetensors):
        dense Llama / Qwen3 style decoders.  Every rank reads only its slices (query / KV heads and MLP columns
        by rows, ``o_proj`` / ``down_proj`` by columns), layer by layer at the first forward, and keeps them on
        the device."""
        root = Path(path)
        config = json.loads((root / "config.json").read_text())
        config = config.get("text_config", config)
        self = cls(config, group=group, device=device, dtype=dtype, resident=True, max_tokens=max_tokens, comm=comm)
        self._checkpoint = _ShardedCheckpoint(root)
        self.layers_counted = True  # a real verifier's states must be the ones a vLLM server hands out for the same ids
        return self

    def embed_weight(self) -> torch.Tensor:
        if self._checkpoint is not None:
            key = self._checkpoint.key("embed_tokens.weight")
            if key is None:
                raise KeyError("the checkpoint holds no embed_tokens.weight")
            return self._checkpoint.read(key).to(device=self.device, dtype=self.dtype)
        return _seeded((self.cfg.vocab_size, self.cfg.hidden_size), 0.02, self.seed * 1000 + 900, self.device, self.dtype)

    def _checkpoint_layer_state(self, idx: int, names: list[str]) -> dict[str, torch.Tensor]:
        """This rank's slices of layer ``idx`` under the layer's own (Hugging Face) tensor names."""
        ck, R, r = self._checkpoint, self.world, self.rank
        state = {}
        for name in names:
            key = ck.key(f"layers.{idx}.{name}")
            if key is None:
                raise KeyError(f"layers.{idx}.{name} is not in the checkpoint at {ck.path}")
            module, kind = name.rsplit(".", 2)[-2:]
            if module in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"):  # column parallel: split the output features
                n = ck._handle(key).get_slice(key).get_shape()[0]  # noqa: SLF001
                state[name] = ck.read(key, rows=(r * n // R, (r + 1) * n // R))
            elif module in ("o_proj", "down_proj"):  # row parallel: split the input features
                if kind == "bias":
                    raise ValueError(f"{name}: a bias on a row-parallel projection is not supported by the tensor-parallel verifier")
                n = ck._handle(key).get_slice(key).get_shape()[1]  # noqa: SLF001
                state[name] = ck.read(key, cols=(r * n // R, (r + 1) * n // R))
            else:  # norms: replicated
                state[name] = ck.read(key)
        return state

    def _slice(self, name: str, full: torch.Tensor) -> torch.Tensor:
        """This rank's part of a full layer tensor."""
        c, R, r = self.cfg, self.world, self.rank
        hd = c.head_dim
        if name.endswith("qkv_proj.weight"):
            nq, nk = c.num_attention_heads * hd, c.num_key_value_heads * hd
            q, k, v = full[:nq], full[nq : nq + nk], full[nq + nk :]
            return torch.cat([t.chunk(R, dim=0)[r] for t in (q, k, v)], dim=0)
        if name.endswith("gate_up_proj.weight"):
            gate, up = full.chunk(2, dim=0)
            return torch.cat([gate.chunk(R, dim=0)[r], up.chunk(R, dim=0)[r]], dim=0)
        if name.endswith(("o_proj.weight", "down_proj.weight")):
            return full.chunk(R, dim=1)[r]
        return full  # norms: replicated

    def _layer(self, idx: int) -> DecoderLayer:
        if idx in self._layers:
            return self._layers[idx]
        layer = DecoderLayer(self.local_cfg, idx)
        own = dict(layer.named_parameters())
        if self._checkpoint is not None:
            # the layer's state dict speaks the checkpoint's names (fused projections are split on save / merged on load)
            layer.load_state_dict(self._checkpoint_layer_state(idx, list(layer.state_dict().keys())), strict=True)
            layer.to(device=self.device, dtype=self.dtype)
        with torch.no_grad():
            for j, (name, shape) in enumerate(self._full_shapes if self._checkpoint is None else []):
                p = own[name]
                if len(shape) == 2 and self.sliced_init:
                    p.data = _seeded(tuple(p.shape), 0.02, ((self.seed * 1000 + idx) * 64 + j) * 16 + self.rank, self.device, self.dtype)
                elif len(shape) == 2:
                    full = _seeded(shape, 0.02, (self.seed * 1000 + idx) * 64 + j, self.device, self.dtype)
                    p.data = self._slice(name, full).contiguous()
                    del full
                else:
                    p.data = p.data.to(device=self.device, dtype=self.dtype)
        if self.comm is not None:
            layer.self_attn.o_proj.row_parallel = self.comm.row_parallel
            layer.mlp.down_proj.row_parallel = self.comm.row_parallel
        if self.resident:
            self._layers[idx] = layer
        return layer

    def _reduce(self, partial: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, layer_ids: list[int], document_ids: torch.Tensor | None = None, position_ids: torch.Tensor | None = None):
        """Same contract as ``RandomVerifier.forward``; every rank of the group calls it with the
        same inputs and gets the same (complete) hidden states."""
        ids = input_ids.reshape(-1).to(self.device)
        T = ids.shape[0]
        doc = document_ids.reshape(-1).to(self.device) if document_ids is not None else torch.zeros(T, dtype=torch.long, device=self.device)
        pos = position_ids.reshape(-1).to(self.device) if position_ids is not None else torch.arange(T, device=self.device)
        lo, hi = causal_document_interval(doc)
        spec = AttnSpec(lo=lo, hi=hi)
        if self.resident:
            if not hasattr(self, "_embed"):
                self._embed = self.embed_weight()
            h = torch.nn.functional.embedding(ids, self._embed)
        else:
            h = torch.nn.functional.embedding(ids, self.embed_weight())
        taken: dict[int, torch.Tensor] = {}
        fused = self.comm is not None
        shift = 1 if self.layers_counted else 0
        if self.layers_counted and 0 in layer_ids:
            taken[0] = h
        for i in range(int(self.cfg.num_hidden_layers)):
            layer = self._layer(i)
            if fused:
                # o_proj / down_proj: product, sum over the ranks and residual add in two kernels; the result
                # alternates between two peer buffers, so what is kept beyond the next call is copied
                h = layer.self_attn(layer.input_layernorm(h), pos, self.rotary, spec, residual=h)
                h = layer.mlp(layer.post_attention_layernorm(h), residual=h)
            else:
                h = h + self._reduce(layer.self_attn(layer.input_layernorm(h), pos, self.rotary, spec))
                h = h + self._reduce(layer.mlp(layer.post_attention_layernorm(h)))
            if i + shift in layer_ids:
                taken[i + shift] = h.clone() if fused else h
            del layer
        if fused:
            h = h.clone()
        return {"hidden_states": torch.cat([taken[i] for i in layer_ids], dim=-1), "verifier_last_hidden_states": h}
