"""Benchmark inputs as files, built with plain PyTorch only.

Both arms of ``bench.py`` (this framework and the unmodified reference) must start
from byte-identical inputs, and the reference arm must not load any code of this
framework.  This module therefore imports nothing but ``torch`` and ``safetensors``:
it writes, under one directory of the temporary folder,

* ``verifier/``          ``config.json`` + ``model.safetensors`` (``model.embed_tokens.weight``,
                          ``lm_head.weight``, ``model.norm.weight`` of a seeded random verifier),
* ``vocab_maps.pt``      ``d2t`` / ``t2d`` for the top-``draft_vocab`` ids of a seeded token stream,
* ``batches_rankR.pt``   the post-collate training batches of rank ``R`` (token ids, loss mask,
                          positions, documents and the hidden states of a plain-PyTorch forward of
                          the random verifier, evaluated one layer at a time),

and returns them as tensors.  ``seeded_draft_init`` gives both arms the same initial values
for the trainable draft weights, keyed by state-dict name.

The batch layout is what the reference's collate function hands its trainer
(src/speculators/train/data.py:344-393; scripts/benchmark.py:187-210 builds the same dict).
"""

from __future__ import annotations

import json
import os
import tempfile
import zlib

import torch
from safetensors.torch import load_file, save_file

__all__ = ["ensure_inputs", "load_batches", "seeded_draft_init", "inputs_dir"]


def inputs_dir(tag: str) -> str:
    return os.path.join(tempfile.gettempdir(), f"sb200_bench_inputs_{tag}")


def _seeded(shape, std: float, seed: int, device, dtype) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def _rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    # x: [T, heads, d]; rotate-half convention
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None, :], torch.cat([ang.sin(), ang.sin()], -1)[:, None, :]
    xf = x.float()
    rot = torch.cat([-xf[..., d // 2 :], xf[..., : d // 2]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


@torch.no_grad()
def _verifier_forward(cfg: dict, ids: torch.Tensor, pos: torch.Tensor, layer_ids: list[int], device, dtype, seed: int = 0):
    """Hidden states of a dense Llama / Qwen3-style decoder with seeded random weights, one layer
    resident at a time.  ``ids`` / ``pos``: [T] (one causal document)."""
    H, heads, kv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or H // heads
    inter, eps, theta = cfg["intermediate_size"], cfg["rms_norm_eps"], float(cfg["rope_theta"])
    qk_norm = cfg.get("model_type") == "qwen3"
    ids, pos = ids.to(device), pos.to(device)
    T = ids.shape[0]
    h = torch.nn.functional.embedding(ids, _seeded((cfg["vocab_size"], H), 0.02, seed * 1000 + 900, device, dtype))
    taken: dict[int, torch.Tensor] = {}
    last_needed = cfg["num_hidden_layers"]
    for i in range(last_needed):
        s = (seed * 1000 + i) * 64
        wq = _seeded((heads * d, H), 0.02, s + 0, device, dtype)
        wk = _seeded((kv * d, H), 0.02, s + 1, device, dtype)
        wv = _seeded((kv * d, H), 0.02, s + 2, device, dtype)
        wo = _seeded((H, heads * d), 0.02, s + 3, device, dtype)
        x = _rms(h, eps)
        q, k, v = (x @ wq.t()).view(T, heads, d), (x @ wk.t()).view(T, kv, d), (x @ wv.t()).view(T, kv, d)
        if qk_norm:
            q, k = _rms(q, eps), _rms(k, eps)
        q, k = _rope(q, pos, theta), _rope(k, pos, theta)
        a = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None], is_causal=True, enable_gqa=True,
        )[0].transpose(0, 1).reshape(T, heads * d)
        h = h + a @ wo.t()
        del wq, wk, wv, wo, q, k, v, a
        wg = _seeded((inter, H), 0.02, s + 4, device, dtype)
        wu = _seeded((inter, H), 0.02, s + 5, device, dtype)
        wd = _seeded((H, inter), 0.02, s + 6, device, dtype)
        x = _rms(h, eps)
        h = h + (torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t())) @ wd.t()
        del wg, wu, wd
        if i in layer_ids:
            taken[i] = h
    return torch.cat([taken[i] for i in layer_ids], dim=-1), h


def _span_mask(T: int, p: float, span: int, gen: torch.Generator) -> torch.Tensor:
    on = torch.rand((T + span - 1) // span, generator=gen) < p
    return on.repeat_interleave(span)[:T]


def _make_batch_mtp(cfg: dict, seq_len: int, seed: int):
    """MTP fine-tuning batch: token ids and the verifier's last hidden states (unit normal, RMS-normalised)."""
    gen = torch.Generator().manual_seed(seed)
    T, H = seq_len, cfg["hidden_size"]
    ids = torch.randint(0, cfg["vocab_size"], (T,), generator=gen)
    mask = _span_mask(T, 0.6, max(1, min(64, T // 32)), gen)
    hs = torch.randn(T, H, generator=gen)
    hs = (hs * torch.rsqrt(hs.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    return {
        "input_ids": ids.unsqueeze(0), "hidden_states": hs.unsqueeze(0).contiguous(), "loss_mask": mask.unsqueeze(0),
        "position_ids": torch.arange(T, dtype=torch.long).unsqueeze(0), "document_ids": torch.zeros(1, T, dtype=torch.long),
    }


def _make_batch(cfg: dict, seq_len: int, layer_ids: list[int], seed: int, device, dtype, verifier_forward: bool):
    gen = torch.Generator().manual_seed(seed)
    T, H = seq_len, cfg["hidden_size"]
    ids = torch.randint(0, cfg["vocab_size"], (T,), generator=gen)
    mask = _span_mask(T, 0.6, max(1, min(64, T // 32)), gen)
    pos = torch.arange(1, T + 1, dtype=torch.long)
    doc = torch.zeros(T, dtype=torch.long)
    if verifier_forward:
        aux, last = _verifier_forward(cfg, ids, pos, layer_ids, device, dtype)
        aux, last = aux.to("cpu", torch.bfloat16), last.to("cpu", torch.bfloat16)
    else:
        aux = torch.randn(T, len(layer_ids) * H, generator=gen).to(torch.bfloat16)
        last = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    return {
        "hidden_states": aux.unsqueeze(0).contiguous(), "input_ids": ids.unsqueeze(0), "verifier_last_hidden_states": last.unsqueeze(0).contiguous(),
        "loss_mask": mask.unsqueeze(0), "position_ids": pos.unsqueeze(0), "document_ids": doc.unsqueeze(0),
    }


def _vocab_maps(vocab_size: int, draft_vocab: int, seq_len: int, seed: int = 0):
    """``d2t`` (draft id -> offset to the verifier id) and ``t2d`` (verifier id kept?) for the
    ``draft_vocab`` most frequent ids of a seeded uniform stream, ties broken by id."""
    gen = torch.Generator().manual_seed(seed + 17)
    stream = torch.randint(0, vocab_size, (64 * seq_len,), generator=gen)
    freq = torch.bincount(stream, minlength=vocab_size)
    order = torch.sort(freq, descending=True, stable=True).indices[:draft_vocab]
    kept = torch.sort(order).values
    t2d = torch.zeros(vocab_size, dtype=torch.bool)
    t2d[kept] = True
    d2t = kept - torch.arange(draft_vocab)
    return d2t, t2d


def ensure_inputs(cfg: dict, tag: str, *, seq_len: int, draft_vocab: int | None, layer_ids: list[int], rank: int, local_rank: int,
                  n_batches: int, device, verifier_forward: bool, barrier, kind: str = "eagle3") -> str:
    """Write whatever is missing of the input files; ``barrier()`` separates the shared files
    (written by local rank 0) from their readers.  Returns the directory."""
    root = inputs_dir(tag)
    os.makedirs(root, exist_ok=True)
    device = torch.device(device)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    vdir = os.path.join(root, "verifier")
    if local_rank == 0 and not os.path.exists(os.path.join(vdir, ".done")):
        os.makedirs(vdir, exist_ok=True)
        with open(os.path.join(vdir, "config.json"), "w") as fh:
            json.dump(cfg, fh, indent=2)
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        save_file(
            {
                "model.embed_tokens.weight": _seeded((V, H), 0.02, 900, device, torch.bfloat16).cpu().contiguous(),
                "lm_head.weight": _seeded((V, H), 0.02, 901, device, torch.bfloat16).cpu().contiguous(),
                "model.norm.weight": torch.ones(H, dtype=torch.bfloat16),
            },
            os.path.join(vdir, "model.safetensors"), metadata={"format": "pt"},
        )
        if draft_vocab:
            d2t, t2d = _vocab_maps(V, draft_vocab, seq_len)
            torch.save({"d2t": d2t, "t2d": t2d}, os.path.join(root, "vocab_maps.pt"))
        open(os.path.join(vdir, ".done"), "w").close()
    mine = os.path.join(root, f"batches_rank{rank}.pt")
    if not os.path.exists(mine):
        if kind == "mtp":
            batches = [_make_batch_mtp(cfg, seq_len, 1000 * rank + i) for i in range(n_batches)]
        else:
            batches = [_make_batch(cfg, seq_len, layer_ids, 1000 * rank + i, device, dtype, verifier_forward) for i in range(n_batches)]
        torch.save(batches, mine + ".tmp")
        os.replace(mine + ".tmp", mine)
    if device.type == "cuda":
        torch.cuda.empty_cache()
    barrier()
    return root


def load_batches(root: str, rank: int, pin: bool):
    batches = torch.load(os.path.join(root, f"batches_rank{rank}.pt"))
    if pin:
        batches = [{k: v.contiguous().pin_memory() for k, v in b.items()} for b in batches]
    return batches


def load_vocab_maps(root: str):
    maps = torch.load(os.path.join(root, "vocab_maps.pt"))
    return maps["d2t"], maps["t2d"]


FROZEN_PREFIXES = ("embed_tokens.", "lm_head.", "verifier_lm_head.", "verifier_norm.", "d2t", "t2d")


def seeded_draft_init(shapes: dict[str, tuple]) -> dict[str, torch.Tensor]:
    """Initial values for the trainable tensors of a draft, from their state-dict names and shapes
    alone: matrices N(0, 0.02) seeded by the CRC of the name, vectors (norm weights) ones.  Names
    that the draft takes from the verifier are left out."""
    out = {}
    for name in sorted(shapes):
        if name.startswith(FROZEN_PREFIXES):
            continue
        shape = tuple(shapes[name])
        if len(shape) >= 2:
            gen = torch.Generator().manual_seed(zlib.crc32(name.encode()))
            out[name] = torch.randn(shape, generator=gen, dtype=torch.float32) * 0.02
        else:
            out[name] = torch.ones(shape, dtype=torch.float32)
    return out


def write_result(tag: str, impl: str, world: int, record: dict) -> None:
    with open(os.path.join(inputs_dir(tag), f"result_{impl}_n{world}.json"), "w") as fh:
        json.dump(record, fh)


def read_result(tag: str, impl: str, world: int) -> dict | None:
    path = os.path.join(inputs_dir(tag), f"result_{impl}_n{world}.json")
    if not os.path.exists(path):
        return None
    try:
        with open(path) as fh:
            return json.load(fh)
    except (OSError, json.JSONDecodeError):
        return None

