"""Expert-parallel token exchange over NVLink peer memory.

The dispatch and combine all-to-alls of a sparse MoE layer (reference:
``speculators/models/mtp`` verifier layers run HF ``Qwen3NextSparseMoeBlock``; expert
parallelism itself has no counterpart there) are done by row kernels that read and write
the other ranks' buffers directly (``ops/csrc/ep_a2a.cu``) instead of a library
all-to-all surrounded by permutations:

* dispatch: every (token, expert) slot is pushed straight to its final place in the
  destination rank's receive buffer — grouped by local expert, then by source rank — so
  the receiver feeds its grouped GEMM without sorting;
* combine: every token pulls its ``k`` expert outputs out of the ranks' buffers and
  forms the routing-weighted sum in the same kernel;
* backward runs the mirrored pattern (push of the weighted output gradient; pull of the
  dispatched rows' gradients); the routing-weight gradient ``<y, dout>`` uses the rows the
  forward pull kept.

Only the per-(rank, expert) token counts (a few hundred integers) travel through the
process group.  Every wait on another rank is a bounded poll that reports through a status
word (:meth:`EpComm.check_status`).

A buffer is only live inside one phase (what autograd needs later is copied out right
after the wait), and every phase ends with a wait on all ranks, so a rank that runs ahead
cannot overwrite rows another rank still reads; two copies used on alternating calls add
slack on top of that.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from speculators_b200 import ops

__all__ = ["EpComm", "EpPlan", "build_plan", "ep_dispatch", "ep_combine"]

_KINDS = ("x", "y", "dy", "dx")  # dispatched rows, expert outputs, their gradients (backward)


@dataclass
class EpPlan:
    """Where every (token, expert) slot of this rank lives on its expert's rank."""

    src_row: torch.Tensor     # int32 [T*k] token index of the slot
    dst_rank: torch.Tensor    # int32 [T*k] rank that owns the slot's expert
    dst_pos: torch.Tensor     # int32 [T*k] row in that rank's receive buffer
    n_recv: int               # rows this rank receives
    max_recv: int             # rows the busiest rank receives (every rank checks it against the capacity)
    local_counts: torch.Tensor  # int64 [num_local] rows per local expert (receive buffer order)
    top_k: int
    parity: int = 0


def build_plan(top_e: torch.Tensor, counts_all: torch.Tensor, rank: int, num_local: int) -> EpPlan:
    """``top_e``: [T, k] global expert ids of this rank's tokens; ``counts_all``: [R, E]
    tokens per (source rank, global expert).  The receive buffer of a rank is ordered by
    (local expert, source rank, order of appearance at the source)."""
    T, k = top_e.shape
    R, E = counts_all.shape
    dev = top_e.device
    flat_e = top_e.reshape(-1).long()
    # first row of every (destination rank, local expert, source rank) block
    per_dest = counts_all.view(R, R, num_local).permute(1, 2, 0).reshape(R, num_local * R)
    base = (per_dest.cumsum(1) - per_dest).view(R, num_local, R)[:, :, rank].reshape(E)
    # order of appearance inside this rank's own (expert) groups
    order = torch.argsort(flat_e, stable=True)
    mine = counts_all[rank]
    start = mine.cumsum(0) - mine
    within = torch.empty_like(flat_e)
    within[order] = torch.arange(flat_e.numel(), device=dev) - start[flat_e[order]]
    mine_cols = counts_all[:, rank * num_local : (rank + 1) * num_local]
    per_rank = counts_all.view(R, R, num_local).sum((0, 2))
    n_recv, max_recv = torch.stack([per_rank[rank], per_rank.max()]).tolist()  # one host read
    return EpPlan(
        src_row=(torch.arange(T * k, device=dev) // k).to(torch.int32),
        dst_rank=(flat_e // num_local).to(torch.int32),
        dst_pos=(base[flat_e] + within).to(torch.int32),
        n_recv=int(n_recv),
        max_recv=int(max_recv),
        local_counts=mine_cols.sum(0),
        top_k=k,
    )


class EpComm:
    """Peer-mapped exchange buffers of one expert-parallel group: :meth:`connect` maps the
    other ranks' buffers through CUDA IPC; :meth:`connect_local` wires several virtual ranks
    of one process to each other (tests)."""

    def __init__(self, group, hidden: int, capacity_rows: int, device: torch.device, *, rank: int | None = None,
                 world: int | None = None, spin_limit: int | None = None):
        if hidden % 8:
            raise ValueError("hidden size must be a multiple of 8")
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        if not 1 <= self.world <= 16:
            raise ValueError("expert-parallel groups of 1..16 ranks are supported")
        self.hidden, self.capacity, self.device = hidden, int(capacity_rows), torch.device(device)
        if spin_limit is None:  # tens of seconds by default (SB200_PEER_WAIT_S), like the optimizer's barriers
            from speculators_b200.parallel.engine import peer_wait_spins

            spin_limit = peer_wait_spins()
        self.spin_limit = int(spin_limit)
        self._nat = ops.native()
        self._seq = 0
        self._calls = 0
        nbytes = self.capacity * hidden * 2
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        with torch.cuda.device(dev_index):
            self._own = {(kind, par): int(self._nat.peer_alloc(nbytes)) for kind in _KINDS for par in (0, 1)}
            self._own_flags = int(self._nat.peer_alloc(16 * 4))
        self.buf = {key: self._nat.peer_tensor(ptr, self.capacity * hidden, torch.bfloat16, dev_index).view(self.capacity, hidden)
                    for key, ptr in self._own.items()}
        self.flags = self._nat.peer_tensor(self._own_flags, 16, torch.int32, dev_index)
        self.flags.zero_()
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._mapped: list[int] = []
        self.ptrs: dict = {}
        self.flag_ptrs: torch.Tensor | None = None

    # ------------------------------------------------------------------ wiring
    def connect(self) -> None:
        """Exchange CUDA IPC handles inside the process group and map every rank's buffers."""
        torch.cuda.synchronize(self.device)
        names = [*self._own.keys(), "flags"]
        mine = {name: self._nat.peer_handle(self._own_flags if name == "flags" else self._own[name]) for name in names}
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        table = {name: [] for name in names}
        for q, handles in enumerate(everyone):
            for name in names:
                if q == self.rank:
                    table[name].append(self._own_flags if name == "flags" else self._own[name])
                else:
                    mapped = int(self._nat.peer_open(handles[name]))
                    self._mapped.append(mapped)
                    table[name].append(mapped)
        self._set_table(table)
        dist.barrier(group=self.group)

    @staticmethod
    def connect_local(comms: list["EpComm"]) -> None:
        """Wire the virtual ranks of one process to each other (same device, plain pointers)."""
        for c in comms:
            table = {name: [o._own[name] for o in comms] for name in c._own}
            table["flags"] = [o._own_flags for o in comms]
            c._set_table(table)

    def _set_table(self, table: dict) -> None:
        self.ptrs = {name: torch.tensor(vals, dtype=torch.int64) for name, vals in table.items() if name != "flags"}
        self.flag_ptrs = torch.tensor(table["flags"], dtype=torch.int64)

    def close(self) -> None:
        for ptr in self._mapped:
            self._nat.peer_close(ptr)
        self._mapped = []
        for ptr in [*self._own.values(), self._own_flags]:
            self._nat.peer_release(ptr)
        self._own = {}

    # ------------------------------------------------------------------ phases
    def next_parity(self) -> int:
        self._calls += 1
        return self._calls & 1

    def _next_seq(self) -> int:
        self._seq += 1
        return self._seq

    def push(self, kind: str, parity: int, src: torch.Tensor, plan: EpPlan, scale=None) -> int:
        """Rows of ``src`` to their slots' places in the ranks' ``kind`` buffers, then publish.
        Returns the sequence number to wait for."""
        seq = self._next_seq()
        self._nat.ep_push(src, plan.src_row, plan.dst_rank, plan.dst_pos, scale, self.ptrs[(kind, parity)], self.capacity,
                          self.counter, self.flag_ptrs, self.rank, self.world, seq)
        return seq

    def signal(self) -> int:
        seq = self._next_seq()
        self._nat.ep_signal(self.flag_ptrs, self.rank, self.world, seq, self.flags)
        return seq

    def wait(self, seq: int) -> None:
        self._nat.ep_wait(self.flags, self.world, seq, self.spin_limit, self.status)

    def pull(self, kind: str, parity: int, plan: EpPlan, weight, n_tokens: int, keep_rows: bool = False):
        """Weighted sum of every token's rows out of the ranks' ``kind`` buffers; with
        ``keep_rows`` also the gathered rows [T*k, H]."""
        out = torch.empty(n_tokens, self.hidden, dtype=torch.bfloat16, device=self.device)
        rows = torch.empty(n_tokens * plan.top_k, self.hidden, dtype=torch.bfloat16, device=self.device) if keep_rows else None
        self._nat.ep_pull(self.ptrs[(kind, parity)], self.capacity, plan.dst_rank, plan.dst_pos, weight, self.world, out, plan.top_k, rows)
        return (out, rows) if keep_rows else out

    def check_status(self, code: int | None = None) -> None:
        """Raise if a wait of the exchange ran out: the rows read after such a wait are stale, so
        training must stop.  ``code``: a value of the status word already copied to the host."""
        if code is None:
            code = int(self.status.item())
        if code:
            raise RuntimeError(f"expert-parallel exchange: a rank did not arrive within the wait budget (status {code})")


class _Dispatch(torch.autograd.Function):
    """x [T, H] -> this rank's received rows [n_recv, H] (copied out of the receive buffer)."""

    @staticmethod
    def forward(ctx, x, comm: EpComm, plan: EpPlan):
        if plan.max_recv > comm.capacity:
            raise RuntimeError(f"expert-parallel receive buffer too small: {plan.max_recv} rows > capacity {comm.capacity}")
        comm.wait(comm.push("x", plan.parity, x.contiguous(), plan))
        ctx.comm, ctx.plan, ctx.n_tokens = comm, plan, x.shape[0]
        return comm.buf[("x", plan.parity)][: plan.n_recv].clone()

    @staticmethod
    def backward(ctx, d_recv):
        comm, plan = ctx.comm, ctx.plan
        comm.buf[("dx", plan.parity)][: plan.n_recv].copy_(d_recv)
        comm.wait(comm.signal())
        ones = None  # weight 1 for every slot
        return comm.pull("dx", plan.parity, plan, ones, ctx.n_tokens), None, None


class _Combine(torch.autograd.Function):
    """Expert outputs of the received rows [n_recv, H] + routing weights [T, k] -> [T, H]."""

    @staticmethod
    def forward(ctx, y_local, top_p, comm: EpComm, plan: EpPlan):
        comm.buf[("y", plan.parity)][: plan.n_recv].copy_(y_local)
        comm.wait(comm.signal())
        w = top_p.reshape(-1).float().contiguous()
        out, rows = comm.pull("y", plan.parity, plan, w, top_p.shape[0], keep_rows=True)
        ctx.comm, ctx.plan = comm, plan
        ctx.save_for_backward(w, rows)
        ctx.p_dtype = top_p.dtype
        ctx.p_shape = top_p.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        comm, plan = ctx.comm, ctx.plan
        w, rows = ctx.saved_tensors
        dout = dout.contiguous()
        comm.wait(comm.push("dy", plan.parity, dout, plan, scale=w))  # weighted output gradient to the experts' ranks
        d_y = comm.buf[("dy", plan.parity)][: plan.n_recv].clone()
        T, k = ctx.p_shape
        d_p = torch.bmm(rows.view(T, k, -1), dout.unsqueeze(-1)).squeeze(-1)  # <y row, dout> per slot
        return d_y, d_p.to(ctx.p_dtype), None, None


def ep_dispatch(x: torch.Tensor, comm: EpComm, plan: EpPlan) -> torch.Tensor:
    return _Dispatch.apply(x, comm, plan)


def ep_combine(y_local: torch.Tensor, top_p: torch.Tensor, comm: EpComm, plan: EpPlan) -> torch.Tensor:
    return _Combine.apply(y_local, top_p, comm, plan)
