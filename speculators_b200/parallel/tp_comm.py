"""Row-parallel products of a tensor-parallel group without a library all-reduce.

A Megatron-style layer ends in a product whose contraction is split over the ranks (``o_proj``,
``down_proj``): every rank holds a partial sum of the whole ``[T, H]`` output, and the reference's
verifier server (vLLM with ``--tensor-parallel-size``, scripts/launch_vllm.py:104-163) all-reduces
it with NCCL.  Here the product and the collective are two kernels that share the work:

1. ``gemm_scatter`` - the tcgen05 GEMM whose epilogue stores every finished tile straight into the
   staging area of the rank that owns those columns (plain stores into peer-mapped memory over
   NVLink, issued while the tensor core works on the next tile), i.e. the reduce-scatter's
   transfer rides under the GEMM;
2. ``tp_reduce_broadcast`` - every rank adds the ``world`` staged slices of its own columns in
   fp32, adds the residual stream's slice, rounds once and writes the slice into every rank's
   output buffer (the all-gather), between two cross-rank barriers.

Buffers live in peer memory (CUDA IPC inside the group, so sub-groups of the job work).  The
output alternates between two buffers, so the residual input of one call may be the output of
the previous one.  Every wait on another rank is bounded and reports through :meth:`check_status`.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from speculators_b200 import ops

__all__ = ["TpComm"]

_STATUS = {61: "a rank never finished its product (opening barrier)", 62: "a rank never wrote its slice (closing barrier)",
           63: "this rank's leading block never released the others"}


class TpComm:
    def __init__(self, group, rows: int, width: int, device: torch.device, *, rank: int | None = None, world: int | None = None,
                 spin_limit: int | None = None):
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        if not 1 <= self.world <= 8:
            raise ValueError("tensor-parallel groups of 1..8 ranks are supported")
        if not self.supported(width, self.world):
            raise ValueError(f"width / world ({width} / {self.world}) must be a multiple of 256")
        self.rows, self.width, self.cols, self.device = int(rows), int(width), width // self.world, torch.device(device)
        if spin_limit is None:
            from speculators_b200.parallel.engine import peer_wait_spins

            spin_limit = peer_wait_spins()
        self.spin_limit = int(spin_limit)
        self._nat = ops.native()
        n = self.rows * self.width
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        words = int(self._nat.tp_allreduce_ctl_words())
        with torch.cuda.device(dev_index):
            self._own = {"stage": int(self._nat.peer_alloc(n * 2)), "out0": int(self._nat.peer_alloc(n * 2)),
                         "out1": int(self._nat.peer_alloc(n * 2)), "ctl": int(self._nat.peer_alloc(words * 4))}
        self.stage = self._nat.peer_tensor(self._own["stage"], n, torch.bfloat16, dev_index)
        self.out = [self._nat.peer_tensor(self._own[k], n, torch.bfloat16, dev_index) for k in ("out0", "out1")]
        self.ctl = self._nat.peer_tensor(self._own["ctl"], words, torch.int32, dev_index)
        self.ctl.zero_()
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._mapped: list[int] = []
        self.ptrs: dict[str, torch.Tensor] = {}
        self.barrier = True
        self._next = 0

    @staticmethod
    def supported(width: int, world: int) -> bool:
        return world >= 1 and width % world == 0 and (width // world) % 256 == 0

    # ------------------------------------------------------------------ wiring
    def connect(self) -> None:
        """Exchange CUDA IPC handles inside the group and map every rank's buffers."""
        torch.cuda.synchronize(self.device)
        mine = {name: self._nat.peer_handle(ptr) for name, ptr in self._own.items()}
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        for name in self._own:
            row = []
            for q, handles in enumerate(everyone):
                if q == self.rank:
                    row.append(self._own[name])
                else:
                    mapped = int(self._nat.peer_open(handles[name]))
                    self._mapped.append(mapped)
                    row.append(mapped)
            self.ptrs[name] = torch.tensor(row, dtype=torch.int64)
        dist.barrier(group=self.group)

    @staticmethod
    def connect_local(comms: list["TpComm"]) -> None:
        """Wire several virtual ranks of one process (tests on one device): they run one after
        another on one stream, so the cross-rank barriers are switched off."""
        for c in comms:
            for name in c._own:  # noqa: SLF001
                c.ptrs[name] = torch.tensor([o._own[name] for o in comms], dtype=torch.int64)  # noqa: SLF001
            c.barrier = False

    # ------------------------------------------------------------------ the two halves
    def scatter_product(self, x: torch.Tensor, w: torch.Tensor) -> None:
        """``x[T, K_local] @ w[width, K_local].T``; the tiles go to their owners' staging areas."""
        if x.shape[0] > self.rows or w.shape[0] != self.width:
            raise ValueError(f"product of {tuple(x.shape)} x {tuple(w.shape)} does not fit the buffers ({self.rows} rows, width {self.width})")
        self._nat.gemm_scatter(x, w, self.ptrs["stage"], self.rank, ops.gemm_status(x.device))

    def reduce_broadcast(self, rows: int, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of the staged products (+ ``residual``) as ``[rows, width]``, complete on every rank."""
        index = self._next
        self._next ^= 1
        if residual is not None and residual.data_ptr() == self.out[index].data_ptr():
            raise ValueError("the residual must not be the buffer this call writes (keep at most one earlier result alive)")
        stage = self.stage[: self.world * rows * self.cols].view(self.world, rows, self.cols)
        self._nat.tp_reduce_broadcast(stage, self.ptrs[f"out{index}"], 0, residual, self.ptrs["ctl"], self.rank, self.barrier, self.status,
                                      self.spin_limit)
        return self.out[index][: rows * self.width].view(rows, self.width)

    def row_parallel(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``sum over ranks of x_r @ w_r.T (+ residual)``, the same on every rank.  The result
        lives in one of two alternating buffers: it stays valid through the next call."""
        x2 = x.reshape(-1, x.shape[-1])
        res2 = residual.reshape(-1, self.width).contiguous() if residual is not None else None
        self.scatter_product(x2, w)
        return self.reduce_broadcast(x2.shape[0], res2).view(*x.shape[:-1], self.width)

    # ------------------------------------------------------------------ status / teardown
    def check_status(self, code: int | None = None) -> None:
        code = int(self.status.item()) if code is None else int(code)
        if code:
            raise RuntimeError(f"tensor-parallel exchange gave up (code {code}): {_STATUS.get(code, 'unknown wait')}")

    def close(self) -> None:
        mapped_any = bool(self._mapped)
        for ptr in self._mapped:
            self._nat.peer_close(ptr)
        self._mapped.clear()
        if mapped_any and dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.group)  # nobody frees a buffer that a peer still has mapped
        self.stage = self.ctl = None
        self.out = []
        for ptr in self._own.values():
            self._nat.peer_release(ptr)
        self._own = {}
