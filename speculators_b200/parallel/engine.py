"""Flat-buffer training engine: mixed precision, data parallelism and the
optimizer in one place.

Layout.  Every trainable parameter of the model becomes a view into one
contiguous *compute* buffer (bf16 on GPU) and its ``.grad`` a view into a parallel
gradient buffer, so backward accumulates straight into memory that is already
laid out for a single collective.  The optimizer keeps fp32 master weights and
AdamW moments for the slice ``[lo, hi)`` of that buffer owned by this rank:

* replicated mode (the reference's DDP, src/speculators/train/trainer.py:323-336):
  every rank owns everything; gradients are all-reduced.
* sharded mode (the reference's ``--fsdp-shard``,
  src/speculators/train/distributed.py:197-216): each rank owns ``1/world`` of the
  buffer; gradients are reduce-scattered, the owner runs AdamW on its slice and
  the refreshed bf16 weights are all-gathered.  Unlike FSDP2, parameters are
  gathered once per optimizer step, not once per layer call, so the ``S``
  TTT passes of EAGLE-3 reuse resident weights; with 180 GB of HBM per GPU the
  resident bf16 copy of a draft model is negligible.

A step is: (sum of squares of the owned gradient slice -> all-reduce of one
scalar) -> fused AdamW with the clip coefficient applied in-kernel -> all-gather.
No value is read back to the host, so the whole step can be captured in a CUDA
graph.  Muon (the reference's default optimizer for 2-D weights,
src/speculators/train/optimizers.py:61-110) assigns whole matrices to ranks: the owner keeps
the fp32 master copy and the momentum, runs the Newton-Schulz update on the package's GEMM and
broadcasts the refreshed bf16 weights; the AdamW tail (norm weights, embeddings) is sharded or
replicated like the plain AdamW mode.

Expert-parallel parameters (tensors marked ``_sb200_local``: the experts a rank holds differ
from rank to rank) live in a third region at the end of the flat buffers that no collective
touches: their gradients are already complete on the owning rank (its experts saw every rank's
tokens through the dispatch), only their squared norm joins the global gradient norm, and the
owner keeps their full AdamW state.  State dicts present them as the stack of all ranks' experts.
"""

from __future__ import annotations

import contextlib
import logging
import math
import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from torch import nn

from speculators_b200.utils.util import nvtx_range

from speculators_b200 import ops

log = logging.getLogger(__name__)

__all__ = ["EngineConfig", "TrainEngine", "peer_wait_seconds", "peer_wait_spins", "split_named_params_for_muon"]

_ALIGN = 128  # elements; keeps every parameter and every shard 16-byte aligned
_ADAMW_NAME_HINTS = ("embed_tokens", "lm_head")


def split_named_params_for_muon(model: nn.Module):
    """(muon, adamw) named-parameter lists: Muon takes trainable 2-D matrices with
    both dims > 1 that are neither embeddings nor LM heads
    (src/speculators/train/optimizers.py:32-58)."""
    muon, adamw = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        is_matrix = p.ndim == 2 and min(p.shape) > 1 and not any(h in name for h in _ADAMW_NAME_HINTS)
        (muon if is_matrix else adamw).append((name, p))
    return muon, adamw


@dataclass
class EngineConfig:
    lr: float = 1e-4
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01
    max_grad_norm: float = 1.0
    optimizer: str = "adamw"  # "adamw" | "muon"
    muon_lr: float = 0.02
    muon_momentum: float = 0.95
    muon_weight_decay: float = 0.1
    muon_ns_steps: int = 5
    muon_adjust_lr_fn: str = "match_rms_adamw"
    compute_dtype: torch.dtype = torch.bfloat16
    shard: bool = False
    # "nccl": reduce-scatter / all-gather through torch.distributed.  "p2p": the sharded
    # step runs as two fused kernels that read peers' gradients and write peers' weights
    # through NVLink peer mappings (single node, AdamW, bf16 compute).  "nvls": the same two
    # kernels, with the bulk transfers going through an NVLink multicast mapping of the
    # buffers (multimem.ld_reduce / multimem.st: the switch adds and replicates).  "auto":
    # nvls on more than two ranks when the system offers multicast, else p2p when it
    # applies, else nccl.
    comm: str = "auto"
    group: object | None = None
    broadcast_from_rank0: bool = True
    extra: dict = field(default_factory=dict)


class TrainEngine:
    def __init__(self, model: nn.Module, config: EngineConfig, device: torch.device | str | None = None):
        self.model = model
        self.cfg = config
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.group = config.group
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(self.group) if self.distributed else 1
        self.rank = dist.get_rank(self.group) if self.distributed else 0
        # Replicated data parallelism (no ``shard``) with AdamW in bf16 on CUDA takes the sharded step too: reduce-scatter +
        # update of 1 / world of the state + all-gather of the weights gives the result of all-reduce + full update
        # on every rank, moves the same bytes, runs as the fused peer-memory kernels where those apply, and holds
        # 1 / world of the optimizer state.  ``SB200_AUTO_SHARD=0`` keeps the all-reduce form.
        auto_shard = (not config.shard and self.world > 1 and self.device.type == "cuda" and config.optimizer == "adamw"
                      and config.compute_dtype == torch.bfloat16 and os.environ.get("SB200_AUTO_SHARD", "1") != "0")
        self.sharded = (bool(config.shard) or auto_shard) and self.world > 1
        self.nvls = False
        self.p2p = self._want_p2p()
        self.step_count = 0
        self._flatten()
        self._init_state()
        self._lazy_zero = self.device.type == "cuda" and os.environ.get("SB200_EAGER_ZERO_GRAD") != "1"
        if self._lazy_zero:
            self._install_lazy_zero_hooks()

    def _want_p2p(self) -> bool:
        import os

        mode = os.environ.get("SB200_COMM", self.cfg.comm)
        if mode not in ("auto", "nvls", "p2p", "nccl"):
            raise ValueError(f"comm must be auto, nvls, p2p or nccl, got {mode!r}")
        self._comm_mode = mode
        applicable = (
            self.sharded and self.device.type == "cuda" and self.cfg.optimizer == "adamw"
            and self.cfg.compute_dtype == torch.bfloat16 and self.world <= 8
        )
        if mode in ("p2p", "nvls") and not applicable:
            raise ValueError(f"comm={mode!r} needs sharded multi-rank CUDA training with AdamW in bf16 on one node (<= 8 ranks)")
        if applicable and any(getattr(p, "_sb200_local", False) for p in self.model.parameters()):
            if mode in ("p2p", "nvls"):
                raise ValueError(f"comm={mode!r} does not cover models with expert-parallel (rank-local) parameters")
            applicable = False  # the fused step reduces the whole buffer; rank-local experts need the region-aware path
        if not applicable or mode == "nccl":
            return False
        reason = self._peer_memory_unavailable()
        if reason is not None:
            if mode in ("p2p", "nvls"):
                raise RuntimeError(f"comm={mode!r} is not available: {reason}")
            log.info("peer-memory optimizer step not used (%s); using the library collectives", reason)
            self._comm_mode = "nccl"
            return False
        return True

    def _peer_memory_unavailable(self) -> str | None:
        """Why the ranks of this group cannot map one another's memory (None: they can).  Every
        rank publishes its host name and device index; the outcome is formed from the gathered
        lists, so all ranks take the same branch."""
        import socket

        mine = (socket.gethostname(), self.device.index if self.device.index is not None else torch.cuda.current_device())
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        if len({h for h, _ in everyone}) > 1:
            return "the ranks are on more than one node"
        ok = all(q == self.rank or d == mine[1] or _can_access_peer(mine[1], d) for q, (_, d) in enumerate(everyone))
        if len({d for _, d in everyone}) < self.world:
            ok = False  # two ranks on one device: kernels that wait on one another must not share a GPU
        answers: list = [None] * self.world
        dist.all_gather_object(answers, bool(ok), group=self.group)
        if not all(answers):
            return "a rank has no peer access to another rank's GPU (or two ranks share one GPU)"
        return None

    def _alloc_flat(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Flat buffer in ordinary allocator memory, or (p2p) in cudaMalloc'ed memory
        that is exported to the peers."""
        if not self.p2p:
            return torch.zeros(numel, dtype=dtype, device=self.device)
        nat = ops.native()
        ptr = nat.peer_alloc(numel * torch.empty((), dtype=dtype).element_size())
        self._peer_local.append(ptr)
        return nat.peer_tensor(ptr, numel, dtype, self.device.index or 0)

    def _alloc_symmetric_pair(self, numel: int, dtype: torch.dtype):
        """(flat_w, flat_g) in torch symmetric memory, mapped on every rank and, where the
        NVSwitch offers it, reachable through one multicast address; ``None`` when that
        is not available.  All ranks take the same branch: the outcome is agreed with an
        all-reduce before anything depends on it."""
        # measured optimizer step for 294 M parameters on 8 GPUs: 1.70 ms through the
        # multicast mapping, 2.78 ms with per-peer loads / stores (every thread touching
        # eight peers), 2.01 ms with NCCL; on 2 GPUs the per-peer path was 1.5 % ahead
        want = self._comm_mode == "nvls" or (self._comm_mode == "auto" and self.world > 2)
        if not self.p2p or not want or os.environ.get("SB200_MULTIMEM", "1") == "0":
            return None
        bufs, handles, err = [], [], None
        try:
            import torch.distributed._symmetric_memory as symm

            grp = self.group if self.group is not None else dist.group.WORLD
            for _ in range(2):
                t = symm.empty(numel, dtype=dtype, device=self.device)
                t.zero_()
                bufs.append(t)
            for t in bufs:
                h = symm.rendezvous(t, grp)
                ptrs = [int(x) for x in h.buffer_ptrs]
                off = t.data_ptr() - ptrs[self.rank]  # the tensor may sit at an offset inside the mapped allocation
                mc = int(h.multicast_ptr)
                if off < 0 or not mc:
                    raise RuntimeError("no NVLink multicast mapping for the buffer")
                handles.append((h, [x + off for x in ptrs], mc + off))
        except Exception as exc:  # noqa: BLE001 - any failure means "use the peer-mapping path"
            err = exc
        agreed = torch.tensor([0 if err is not None else 1], device=self.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)
        if int(agreed.item()) == 0:
            if self._comm_mode == "nvls":
                raise RuntimeError(f"comm='nvls' is not available on this system: {err or 'another rank failed'}")
            log.info("NVLink multicast not used (%s)", err or "another rank failed")
            self._multicast_refused = self.world > 2 and self._comm_mode == "auto"
            return None
        self._symm_handles = handles  # keeps the mappings alive
        return bufs[0], bufs[1]

    def _exchange(self, local_ptr: int) -> list[int]:
        """All ranks publish the IPC handle of ``local_ptr``; returns the address of
        every rank's buffer as mapped into this process (own buffer: the local address)."""
        nat = ops.native()
        handles: list = [None] * self.world
        dist.all_gather_object(handles, nat.peer_handle(local_ptr), group=self.group)
        out = []
        for q, h in enumerate(handles):
            if q == self.rank:
                out.append(local_ptr)
            else:
                mapped = nat.peer_open(h)
                self._peer_mapped.append(mapped)
                out.append(mapped)
        return out

    # ------------------------------------------------------------------ layout
    def _flatten(self) -> None:
        cfg, dev = self.cfg, self.device
        model = self.model
        # frozen tensors: move + cast, they never enter the flat buffers
        for p in model.parameters():
            if not p.requires_grad:
                p.data = p.data.to(device=dev, dtype=cfg.compute_dtype if p.is_floating_point() else p.dtype)
        for mod in model.modules():
            for key, buf in list(mod._buffers.items()):  # noqa: SLF001
                if buf is not None:
                    mod._buffers[key] = buf.to(dev)  # noqa: SLF001
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not named:
            raise ValueError("No trainable parameters found to optimize.")
        use_muon = cfg.optimizer == "muon"
        muon_names = {n for n, _ in split_named_params_for_muon(model)[0]} if use_muon else set()
        local_names = {n for n, p in named if getattr(p, "_sb200_local", False)} if self.world > 1 else set()
        muon_names -= local_names
        # Muon matrices first, then the AdamW tail, then the rank-local (expert-parallel) tensors
        named.sort(key=lambda np_: 0 if np_[0] in muon_names else (2 if np_[0] in local_names else 1))
        self.names: list[str] = []
        self.params: list[nn.Parameter] = []
        self.offsets: list[int] = []
        off = 0
        self.muon_end = 0
        unit = _ALIGN * self.world
        self.shared_end = -1
        for name, p in named:
            if muon_names and name not in muon_names and self.muon_end == 0 and off > 0:
                # first tensor of the AdamW tail: the matrix region ends on a shard-unit boundary,
                # so the tail divides evenly among the ranks
                off = self.muon_end = (off + unit - 1) // unit * unit
            if name in local_names and self.shared_end < 0:
                if muon_names and self.muon_end == 0:
                    off = self.muon_end = (off + unit - 1) // unit * unit
                off = (off + unit - 1) // unit * unit
                if off == self.muon_end:
                    off += unit
                self.shared_end = off  # everything before is replicated (or sharded) across the ranks
            self.names.append(name)
            self.params.append(p)
            self.offsets.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        if self.shared_end < 0:
            if muon_names and self.muon_end == 0:
                off = self.muon_end = (off + unit - 1) // unit * unit  # matrices only
            self.total = (off + unit - 1) // unit * unit
            if self.total == self.muon_end:
                self.total += unit  # keeps the tail slice non-empty
            self.shared_end = self.total
        else:
            self.total = (off + _ALIGN - 1) // _ALIGN * _ALIGN
        self.local_names = local_names
        self._peer_local: list[int] = []
        self._peer_mapped: list[int] = []
        self._symm_handles = None
        pair = self._alloc_symmetric_pair(self.total, cfg.compute_dtype)
        if pair is None and getattr(self, "_multicast_refused", False):
            # measured at 8 ranks: per-peer loads / stores 2.78 ms, library collectives 2.01 ms
            log.info("NVLink multicast is not available on more than two ranks; using the library collectives")
            self.p2p = False
            self._comm_mode = "nccl"
        if pair is not None:
            self.flat_w, self.flat_g = pair
        else:
            self.flat_w = self._alloc_flat(self.total, cfg.compute_dtype)
            self.flat_g = self._alloc_flat(self.total, cfg.compute_dtype)
        init32 = torch.zeros(self.total, dtype=torch.float32, device=dev)
        for p, o in zip(self.params, self.offsets):
            init32[o : o + p.numel()].copy_(p.data.detach().reshape(-1).to(device=dev, dtype=torch.float32))
        if self.distributed and cfg.broadcast_from_rank0:
            dist.broadcast(init32[: self.shared_end], src=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
            for p in model.parameters():  # frozen weights too: every rank trains the same model
                if not p.requires_grad:
                    dist.broadcast(p.data, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
        self.flat_w.copy_(init32)
        for p, o in zip(self.params, self.offsets):
            p.data = self.flat_w[o : o + p.numel()].view(p.shape)
            p.grad = self.flat_g[o : o + p.numel()].view(p.shape)
            if p.ndim == 2:  # ops.linear accumulates weight gradients straight into this view
                p._flat_grad = p.grad
        self._init32 = init32

    def _init_state(self) -> None:
        # [lo, hi): the slice of the flat buffer whose AdamW state this rank holds.  With Muon the
        # matrix region [0, muon_end) is not part of it: whole matrices are owned by ranks instead
        # (``_init_muon``) and the AdamW slice covers the tail only.
        first = self.muon_end
        if self.sharded:
            per = (self.shared_end - first) // self.world
            self.lo, self.hi = first + self.rank * per, first + (self.rank + 1) * per
        else:
            self.lo, self.hi = first, self.shared_end
        n = self.hi - self.lo
        dev = self.device
        fp32_compute = self.cfg.compute_dtype == torch.float32
        self._init_muon(fp32_compute)
        # with fp32 compute weights the flat buffer *is* the master copy
        self.master = self.flat_w[self.lo : self.hi] if fp32_compute else self._init32[self.lo : self.hi].clone()
        n_local = self.total - self.shared_end
        self.local_master = self.local_exp_avg = self.local_exp_avg_sq = None
        if n_local:
            a, b = self.shared_end, self.total
            self.local_master = self.flat_w[a:b] if fp32_compute else self._init32[a:b].clone()
            self.local_exp_avg = torch.zeros(n_local, dtype=torch.float32, device=dev)
            self.local_exp_avg_sq = torch.zeros(n_local, dtype=torch.float32, device=dev)
            self.local_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        del self._init32
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.hyper = torch.zeros(ops.HYPER_LEN, dtype=torch.float32, device=dev)
        self.grad_shard = (
            torch.zeros(n, dtype=self.cfg.compute_dtype, device=dev) if self.sharded else self.flat_g
        )
        self.base_lr = self.cfg.lr
        self.base_muon_lr = self.cfg.muon_lr
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.p2p:
            nat = ops.native()
            ctl = nat.peer_alloc(int(nat.fused_optim_ctl_words()) * 4)
            self._peer_local.append(ctl)
            self._g_mc = self._w_mc = 0
            if self._symm_handles is not None:
                (_, w_ptrs, w_mc), (_, g_ptrs, g_mc) = self._symm_handles
                self._g_ptrs = torch.tensor(g_ptrs, dtype=torch.int64)
                self._w_ptrs = torch.tensor(w_ptrs, dtype=torch.int64)
                self._g_mc, self._w_mc = g_mc, w_mc
            else:
                self._g_ptrs = torch.tensor(self._exchange(self.flat_g.data_ptr()), dtype=torch.int64)
                self._w_ptrs = torch.tensor(self._exchange(self.flat_w.data_ptr()), dtype=torch.int64)
            self._ctl_ptrs = torch.tensor(self._exchange(ctl), dtype=torch.int64)
            self.nvls = bool(self._g_mc)
            self.grad_reduced = torch.zeros(n, dtype=torch.float32, device=dev)
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ step
    def zero_grad(self) -> None:
        """Clear the gradient buffer.  On CUDA the matrices (almost all of the buffer) are
        not written: they are flagged ``_grad_fresh`` and whoever produces their first
        gradient of the step stores it instead of accumulating (``ops.linear``'s weight
        gradient GEMM, or the hook below for gradients that arrive through autograd's own
        accumulation); ``apply`` clears the ones nothing touched."""
        lazy = self._lazy_zero
        if not lazy:
            self.flat_g.zero_()
        for p, o in zip(self.params, self.offsets):  # re-attach if something replaced .grad
            if p.grad is None or p.grad.data_ptr() != self.flat_g.data_ptr() + o * self.flat_g.element_size():
                p.grad = self.flat_g[o : o + p.numel()].view(p.shape)
                if p.ndim == 2:
                    p._flat_grad = p.grad
            if lazy:
                if p.ndim == 2:
                    p._grad_fresh = True
                else:
                    p.grad.zero_()

    def _install_lazy_zero_hooks(self) -> None:
        def make(p):
            def on_grad(g):
                if getattr(p, "_grad_fresh", False):
                    p._grad_fresh = False
                    p._flat_grad.zero_()
                return g

            return on_grad

        for p in self.params:
            if p.ndim == 2:
                p._grad_fresh = False
                p.register_hook(make(p))

    def mark_grads_written(self) -> None:
        """Call after writing gradients into ``flat_g`` / ``p.grad`` directly (not through
        backward): tells ``apply`` that the matrices' regions hold this step's gradients."""
        for p in self.params:
            if p.ndim == 2:
                p._grad_fresh = False

    def _settle_untouched_grads(self) -> None:
        for p in self.params:
            if p.ndim == 2 and getattr(p, "_grad_fresh", False):
                p._grad_fresh = False
                p._flat_grad.zero_()

    def prepare_hyper(self, lr: float | None = None) -> None:
        """Host side of a step: bump the step counter and stage lr / bias corrections
        (a one-block kernel that takes them by value).  Call before ``apply`` (or before a graph
        replay that contains ``apply``)."""
        self.step_count += 1
        b1, b2 = self.cfg.betas
        lr = self.base_lr if lr is None else lr
        vals = [
            lr, b1, b2, self.cfg.eps, self.cfg.weight_decay,
            1.0 - b1**self.step_count, 1.0 - b2**self.step_count,
            self.cfg.max_grad_norm if self.cfg.max_grad_norm else 0.0,
            1.0 / self.world,
        ]
        if self.hyper.is_cuda:
            # by-value kernel arguments: a pinned staging row would be overwritten by
            # the next call while this step's copy is still queued
            ops.native().set_hyper(self.hyper, vals)
        else:
            self.hyper[: len(vals)] = torch.tensor(vals, dtype=torch.float32)

    def apply(self) -> None:
        """Device side of a step (capturable): reduce, norm, update, gather."""
        if self._lazy_zero:
            self._settle_untouched_grads()
        if self.p2p:
            ops.native().fused_sharded_adamw(
                self.world, self.rank, self.hi - self.lo, self._g_ptrs, self._w_ptrs, self._ctl_ptrs, self._g_mc, self._w_mc,
                self.master, self.exp_avg,
                self.exp_avg_sq, self.grad_reduced, self.hyper, self.status, peer_wait_spins(),
            )
            return
        multi = self.distributed and self.world > 1
        w16 = None if self.cfg.compute_dtype == torch.float32 else self.flat_w[self.lo : self.hi]
        shared_g, shared_w = self.flat_g[: self.shared_end], self.flat_w[: self.shared_end]  # the whole buffers unless experts are rank-local
        if self.muon_items:
            # Muon: every rank needs whole reduced matrices for the ones it owns, so the gradient
            # buffer is all-reduced; the norm is then the same local reduction on every rank
            if multi:
                with nvtx_range("grad reduce"), self._comm_timed():
                    dist.all_reduce(shared_g, op=dist.ReduceOp.SUM, group=self.group)
            ops.sum_of_squares(shared_g, self.norm_sq, accumulate=False)
            self._add_local_norm()
            self._muon_update(self.flat_g)
            ops.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, self.flat_g[self.lo : self.hi], w16, self.hyper, self.norm_sq)
            self._local_update()
            if multi:
                with nvtx_range("weight broadcast"), self._comm_timed():
                    self._muon_broadcast(self.flat_w)
                    if self.sharded:
                        dist.all_gather_into_tensor(self.flat_w[self.muon_end : self.shared_end], self.flat_w[self.lo : self.hi], group=self.group)
            return
        if multi:
            with nvtx_range("grad reduce"), self._comm_timed():
                if self.sharded:
                    dist.reduce_scatter_tensor(self.grad_shard, shared_g, op=dist.ReduceOp.SUM, group=self.group)
                else:
                    dist.all_reduce(shared_g, op=dist.ReduceOp.SUM, group=self.group)
        g = self.grad_shard if self.sharded else shared_g
        ops.sum_of_squares(g, self.norm_sq, accumulate=False)
        if self.sharded:
            if self.local_master is not None:  # one collective for both contributions
                ops.sum_of_squares(self.flat_g[self.shared_end :], self.norm_sq, accumulate=True)
            dist.all_reduce(self.norm_sq, op=dist.ReduceOp.SUM, group=self.group)
        else:
            self._add_local_norm()
        ops.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, g, w16, self.hyper, self.norm_sq)
        self._local_update()
        if self.sharded:
            with nvtx_range("weight all-gather"), self._comm_timed():
                dist.all_gather_into_tensor(shared_w, self.flat_w[self.lo : self.hi], group=self.group)

    def _add_local_norm(self) -> None:
        """Replicated-gradient modes: add the squared norm of every rank's local (expert) gradients
        to the global figure (the shared part is already the same on every rank)."""
        if self.local_master is None:
            return
        ops.sum_of_squares(self.flat_g[self.shared_end :], self.local_sq, accumulate=False)
        if self.distributed and self.world > 1:
            dist.all_reduce(self.local_sq, op=dist.ReduceOp.SUM, group=self.group)
        self.norm_sq += self.local_sq

    def _local_update(self) -> None:
        """AdamW over the rank-local region (full state on the owner, no collective)."""
        if self.local_master is None:
            return
        w16 = None if self.cfg.compute_dtype == torch.float32 else self.flat_w[self.shared_end :]
        ops.adamw_step_(self.local_master, self.local_exp_avg, self.local_exp_avg_sq, self.flat_g[self.shared_end :], w16, self.hyper, self.norm_sq)

    # ------------------------------------------------------------------ exposed communication
    def account_comm(self, enabled: bool) -> None:
        """Time the collectives of the next ``apply`` calls with CUDA events (library-collective
        path; they run on the training stream, so all of their time is exposed).  In the fused
        peer-memory modes the transfers happen inside the optimizer kernel and are part of its
        time.  Not usable while the step is being captured into a CUDA graph."""
        self._comm_events = [] if enabled else None

    @contextlib.contextmanager
    def _comm_timed(self):
        events = getattr(self, "_comm_events", None)
        if events is None or not self.flat_g.is_cuda or torch.cuda.is_current_stream_capturing():
            yield
            return
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        yield
        stop.record()
        events.append((start, stop))

    def exposed_comm_ms(self) -> float | None:
        """Milliseconds the collectives timed since ``account_comm(True)`` took (synchronises on
        their events) and clears the list; ``None`` when nothing was timed."""
        events = getattr(self, "_comm_events", None)
        if not events:
            return None
        total = 0.0
        for start, stop in events:
            stop.synchronize()
            total += start.elapsed_time(stop)
        self._comm_events = []
        return total

    def step(self, lr: float | None = None) -> None:
        self.prepare_hyper(lr)
        self.apply()

    # ------------------------------------------------------------------ muon
    def _init_muon(self, fp32_compute: bool) -> None:
        """Ownership of the Muon matrices.  Newton-Schulz needs a whole matrix, so matrices are
        not cut at shard boundaries: each is assigned to one rank (largest cost first onto the
        least loaded rank, cost = the iteration's GEMM work), which keeps its fp32 master copy and
        momentum, computes its update and broadcasts the refreshed weights.  The same assignment
        is used with and without ``shard``: the result is identical to every rank updating every
        matrix, at 1/world of the work and of the state."""
        self.muon_items: list[tuple[int, str, nn.Parameter, int]] = [
            (i, name, p, o) for i, (name, p, o) in enumerate(zip(self.names, self.params, self.offsets)) if o < self.muon_end
        ]
        self.muon_owner: dict[int, int] = {}
        self.muon_state: dict[int, dict[str, torch.Tensor]] = {}
        if not self.muon_items:
            return
        load = [0.0] * self.world

        def cost(p):
            m, n = min(p.shape), max(p.shape)
            return 4.0 * m * m * n + 2.0 * m**3

        for i, _name, p, _o in sorted(self.muon_items, key=lambda it: (-cost(it[2]), it[0])):
            r = min(range(self.world), key=lambda q: (load[q], q))
            self.muon_owner[i] = r
            load[r] += cost(p)
        for i, _name, p, o in self.muon_items:
            if self.muon_owner[i] != self.rank:
                continue
            n = p.numel()
            master = self.flat_w[o : o + n].view(p.shape) if fp32_compute else self._init32[o : o + n].clone().view(p.shape)
            self.muon_state[i] = {"master": master, "momentum": torch.zeros(p.shape, dtype=torch.float32, device=self.device)}
        if self.device.type == "cuda":
            self._muon_sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
            self._muon_partial = torch.zeros(ops.native().sumsq_num_partials(), dtype=torch.float32, device=self.device)

    def _muon_update(self, g: torch.Tensor) -> None:
        """Momentum + Newton-Schulz orthogonalised update of the matrices this rank owns.
        Same semantics as ``torch.optim.Muon``: nesterov momentum, quintic NS iteration,
        decoupled weight decay and the ``match_rms_adamw`` learning-rate adjustment
        ``0.2 * sqrt(max(m, n))``.  On CUDA the element-wise parts are two kernels (clip + momentum
        + nesterov + bf16 cast + squared norm; decay + update + bf16 cast) and the iteration runs
        on the package's GEMM with transposed operands read in place."""
        cfg = self.cfg
        cuda = self.device.type == "cuda" and cfg.compute_dtype == torch.bfloat16
        lr_ratio = self.base_muon_lr / max(self.base_lr, 1e-30)  # the matrix group follows the AdamW group's schedule
        if not cuda:
            coef_scale = 1.0 / self.world
            total_norm = coef_scale * self.norm_sq.sqrt()
            clip = torch.clamp(cfg.max_grad_norm / (total_norm + 1e-6), max=1.0) if cfg.max_grad_norm else torch.ones_like(total_norm)
        for i, _name, p, o in self.muon_items:
            state = self.muon_state.get(i)
            if state is None:
                continue
            n = p.numel()
            rows, cols = p.shape
            adj = 0.2 * math.sqrt(max(rows, cols)) if cfg.muon_adjust_lr_fn == "match_rms_adamw" else math.sqrt(max(1.0, rows / cols))
            if cuda:
                nat = ops.native()
                upd = torch.empty(p.shape, dtype=torch.bfloat16, device=self.device)
                nat.muon_momentum(g[o : o + n], state["momentum"].view(-1), upd.view(-1), self.hyper, self.norm_sq,
                                  cfg.muon_momentum, True, self._muon_partial, self._muon_sumsq)
                upd = _newton_schulz(upd * (1.0 / (self._muon_sumsq.sqrt() + 1e-7)).to(torch.bfloat16), cfg.muon_ns_steps, normalise=False)
                nat.muon_apply(state["master"].view(-1), upd.reshape(-1), self.flat_w[o : o + n], self.hyper, lr_ratio,
                               cfg.muon_weight_decay, adj)
                continue
            grad = g[o : o + n].view(p.shape).float() * (coef_scale * clip)
            buf = state["momentum"]
            buf.lerp_(grad, 1 - cfg.muon_momentum)
            update = _newton_schulz(grad.lerp(buf, cfg.muon_momentum), cfg.muon_ns_steps)
            lr = self.hyper[0] * lr_ratio
            master = state["master"]
            master.mul_(1 - lr * cfg.muon_weight_decay)
            master.sub_(update * (lr * adj))
            if self.cfg.compute_dtype != torch.float32:
                self.flat_w[o : o + n].view(p.shape).copy_(master)

    def _muon_broadcast(self, flat: torch.Tensor) -> None:
        """Every matrix region of ``flat`` from its owner to all ranks (asynchronous, waited
        together)."""
        work = []
        for i, _name, p, o in self.muon_items:
            src = self.muon_owner[i]
            if self.group is not None:
                src = dist.get_global_rank(self.group, src)
            work.append(dist.broadcast(flat[o : o + p.numel()], src=src, group=self.group, async_op=True))
        for w in work:
            w.wait()

    def _muon_full(self, key: str, first_rank_only: bool = False) -> dict[int, torch.Tensor | None]:
        """``key`` ("master" / "momentum") of every Muon matrix as full fp32 tensors: on every
        rank, or on the group's first rank only (``None`` elsewhere)."""
        out: dict[int, torch.Tensor | None] = {}
        multi = self.distributed and self.world > 1
        for i, _name, p, _o in self.muon_items:
            own = self.muon_state.get(i)
            t = own[key].detach().clone().float() if own is not None else torch.empty(p.shape, dtype=torch.float32, device=self.device)
            if multi:
                src = self.muon_owner[i]
                dist.broadcast(t, src=dist.get_global_rank(self.group, src) if self.group is not None else src, group=self.group)
            out[i] = None if (first_rank_only and self.rank != 0) else t
        return out

    def check_status(self, code: int | None = None) -> None:
        """Raise if a bounded device-side wait of the fused step ran out (a peer did
        not arrive).  A step whose wait ran out applied no update on this rank and the ranks'
        barrier generations no longer pair up, so training must stop here, not continue.
        Without ``code`` this reads one int from the device, so call it where a host sync is
        acceptable; the trainer passes the value it copied out with its step record."""
        if code is None:
            code = int(self.status.item())
        if code != 0:
            names = {11: "gradient barrier", 12: "norm barrier", 13: "closing barrier", 14: "local release"}
            raise RuntimeError(
                f"fused optimizer step timed out waiting at the {names.get(code, code)}: a peer rank did not arrive within "
                f"{peer_wait_seconds():.0f} s (SB200_PEER_WAIT_S); the step was not applied on rank {self.rank}"
            )

    def close(self) -> None:
        """Unmap peers' buffers and free exported memory (p2p mode)."""
        if getattr(self, "_peer_mapped", None) or getattr(self, "_peer_local", None):
            nat = ops.native()
            if self.distributed:
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
            for ptr in self._peer_mapped:
                nat.peer_close(ptr)
            self._peer_mapped = []

    # ------------------------------------------------------------------ state
    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last ``apply`` (device scalar)."""
        return self.norm_sq.sqrt() / self.world

    def _gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        if not self.sharded:
            return shard
        full = torch.empty(self.shared_end - self.muon_end, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def _gather_to_first(self, shard: torch.Tensor) -> torch.Tensor | None:
        """The full tensor on the group's first rank (``None`` elsewhere): only the writer of a
        checkpoint pays the memory and the device-to-host copy."""
        if not self.sharded:
            return shard
        dst = dist.get_global_rank(self.group, 0) if self.group is not None else 0
        if self.rank == 0:
            full = torch.empty(self.shared_end - self.muon_end, dtype=shard.dtype, device=shard.device)
            dist.gather(shard.contiguous(), list(full.chunk(self.world)), dst=dst, group=self.group)
            return full
        dist.gather(shard.contiguous(), None, dst=dst, group=self.group)
        return None

    def _local_stacks(self, region: torch.Tensor | None) -> dict[str, torch.Tensor]:
        """Rank-local tensors of ``region`` (a ``[shared_end, total)`` sized buffer) as the stack of all
        ranks' pieces along dim 0, keyed by parameter name (collective; every rank gets the result)."""
        out: dict[str, torch.Tensor] = {}
        if region is None:
            return out
        for name, p, o in zip(self.names, self.params, self.offsets):
            if name not in self.local_names:
                continue
            mine = region[o - self.shared_end : o - self.shared_end + p.numel()].view(p.shape).float().contiguous()
            full = torch.empty((self.world * p.shape[0], *p.shape[1:]), dtype=torch.float32, device=mine.device)
            dist.all_gather_into_tensor(full, mine, group=self.group)
            out[name] = full
        return out

    def optimizer_state_dict(self, first_rank_only: bool = False) -> dict:
        """Full (unsharded) optimizer state keyed by parameter name; every rank participates in
        the gathers.  With ``first_rank_only`` the tensors are assembled on the group's first
        rank alone and the other ranks get a dict without ``state`` entries."""
        gather = self._gather_to_first if first_rank_only else self._gather_full
        master, m, v = (gather(t) for t in (self.master, self.exp_avg, self.exp_avg_sq))
        mu_master, mu_mom = self._muon_full("master", first_rank_only), self._muon_full("momentum", first_rank_only)
        stacks = {key: self._local_stacks(t) for key, t in (("master", self.local_master), ("exp_avg", self.local_exp_avg), ("exp_avg_sq", self.local_exp_avg_sq))}
        if master is None or (first_rank_only and self.rank != 0 and self.distributed and self.world > 1):
            return {"step": self.step_count, "optimizer": self.cfg.optimizer, "state": {}}
        state = {}
        base = self.muon_end  # the gathered AdamW tensors start at the end of the matrix region
        for i, (name, p, o) in enumerate(zip(self.names, self.params, self.offsets)):
            n = p.numel()
            if i in mu_master:  # a Muon matrix: the momentum sits in "exp_avg", there is no second moment
                state[name] = {"master": mu_master[i].cpu(), "exp_avg": mu_mom[i].cpu(), "exp_avg_sq": torch.zeros(p.shape)}
                continue
            if name in self.local_names:  # the stack of every rank's experts
                state[name] = {key: stacks[key][name].cpu() for key in stacks}
                continue
            a = o - base
            state[name] = {
                "master": master[a : a + n].view(p.shape).cpu().clone(),
                "exp_avg": m[a : a + n].view(p.shape).cpu().clone(),
                "exp_avg_sq": v[a : a + n].view(p.shape).cpu().clone(),
            }
        return {"step": self.step_count, "optimizer": self.cfg.optimizer, "state": state}

    def load_optimizer_state_dict(self, sd: dict) -> None:
        """Restore ``optimizer_state_dict`` output.  A ``torch.optim`` state dict (integer keys
        plus ``param_groups``: what the reference's checkpoints hold) is a different format: it is
        not mapped, the optimizer starts fresh and a warning says so."""
        if "param_groups" in sd or any(isinstance(k, int) for k in sd.get("state", {})):
            log.warning(
                "optimizer state is in torch.optim format (integer parameter indices + param_groups), not this engine's "
                "name-keyed format: moments and step count are NOT restored; the optimizer starts fresh from the loaded weights."
            )
            return
        self.step_count = int(sd.get("step", 0))
        if not any(name in sd.get("state", {}) for name in self.names):
            log.warning("optimizer state matches none of the %d trainable parameter names: nothing restored.", len(self.names))
        for i, (name, p, o) in enumerate(zip(self.names, self.params, self.offsets)):
            entry = sd["state"].get(name)
            if entry is None:
                continue
            if o < self.muon_end:
                own = self.muon_state.get(i)
                if own is not None:
                    own["master"].copy_(entry["master"].reshape(p.shape).float().to(self.device))
                    own["momentum"].copy_(entry["exp_avg"].reshape(p.shape).float().to(self.device))
                continue
            if name in self.local_names:  # this rank's slice of the stacked experts
                a = o - self.shared_end
                for key, dst in (("master", self.local_master), ("exp_avg", self.local_exp_avg), ("exp_avg_sq", self.local_exp_avg_sq)):
                    piece = entry[key].float().chunk(self.world, dim=0)[self.rank] if entry[key].shape[0] == self.world * p.shape[0] else entry[key].float()
                    dst[a : a + p.numel()].copy_(piece.reshape(-1).to(self.device))
                continue
            n = p.numel()
            a, b = max(o, self.lo), min(o + n, self.hi)
            if a >= b:
                continue
            for key, dst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                src = entry[key].reshape(-1).float()[a - o : b - o].to(self.device)
                dst[a - self.lo : b - self.lo].copy_(src)
        self.sync_compute_weights()

    def sync_compute_weights(self) -> None:
        """Refresh the compute buffer from the master weights (after loading state)."""
        if self.cfg.compute_dtype != torch.float32:
            self.flat_w[self.lo : self.hi].copy_(self.master)
            if self.local_master is not None:
                self.flat_w[self.shared_end :].copy_(self.local_master)
            for i, _name, p, o in self.muon_items:
                if i in self.muon_state:
                    self.flat_w[o : o + p.numel()].view(p.shape).copy_(self.muon_state[i]["master"])
        if self.muon_items and self.distributed and self.world > 1:
            self._muon_broadcast(self.flat_w)
        if self.sharded:
            dist.all_gather_into_tensor(self.flat_w[self.muon_end : self.shared_end], self.flat_w[self.lo : self.hi].clone(), group=self.group)

    def load_model_weights_into_master(self) -> None:
        """After ``model.load_state_dict`` wrote new values through the parameter
        views, make them the master copy."""
        if self.cfg.compute_dtype != torch.float32:
            self.master.copy_(self.flat_w[self.lo : self.hi])
            if self.local_master is not None:
                self.local_master.copy_(self.flat_w[self.shared_end :])
            for i, _name, p, o in self.muon_items:
                if i in self.muon_state:
                    self.muon_state[i]["master"].copy_(self.flat_w[o : o + p.numel()].view(p.shape))

    def master_state_dict(self) -> dict[str, torch.Tensor]:
        """fp32 master weights keyed by parameter name (full tensors, on every rank)."""
        master = self._gather_full(self.master)
        mu = self._muon_full("master")
        local = self._local_stacks(self.local_master)
        base = self.muon_end
        return {
            name: (mu[i] if i in mu else local[name] if name in local else master[o - base : o - base + p.numel()].view(p.shape).clone())
            for i, (name, p, o) in enumerate(zip(self.names, self.params, self.offsets))
        }


def peer_wait_seconds() -> float:
    """Budget of every cross-rank wait inside the peer-memory kernels (optimizer barriers,
    expert-parallel exchange).  The library collectives they replace tolerate minutes of rank
    skew (a stalled hidden-state fetch, a one-sided graph capture, logging on rank 0), so the
    default is tens of seconds; it stays bounded so that a lost peer ends in an error."""
    try:
        return min(240.0, max(0.001, float(os.environ.get("SB200_PEER_WAIT_S", "30"))))
    except ValueError:
        return 30.0


def peer_wait_spins(per_second: int = 1 << 24) -> int:
    """The budget as poll iterations (one poll plus a 64 ns back-off is about 60 ns)."""
    return int(min(0xFFFFFFF0, max(1, peer_wait_seconds() * per_second)))


def _can_access_peer(a: int, b: int) -> bool:
    try:
        return bool(torch.cuda.can_device_access_peer(a, b))
    except Exception:  # noqa: BLE001 - an unknown device index counts as "no"
        return False


def _newton_schulz(g: torch.Tensor, steps: int, normalise: bool = True) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal factor of ``g``.  The Gram matrix
    is formed on the short side without materialising a transpose: ``X X^T`` for a wide matrix,
    ``X^T X`` for a tall one (then ``X <- a X + X B`` instead of ``a X + B X``)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.bfloat16() if g.is_cuda else g.clone()
    if normalise:
        x = x / (x.norm() + 1e-7)
    tall = x.shape[0] > x.shape[1]
    for _ in range(steps):
        gram = ops.matmul_tn(x, x) if tall else ops.matmul_nt(x, x)
        poly = b * gram + c * ops.matmul_nn(gram, gram)
        nxt = a * x
        x = ops.matmul_nn(x, poly, out=nxt, accumulate=True) if tall else ops.matmul_nn(poly, x, out=nxt, accumulate=True)
    return x.to(g.dtype)
