"""Expert parallelism over NVLink peer memory.

Each rank of the group owns ``E / world`` experts of every mixture-of-experts layer and routes its
own tokens. The all-to-all exchanges are folded into the permutation kernels (``csrc/ep.cu``):

* ``push_rows``: the rank that owns a token stores the token's row directly into the expert-
  contiguous, tile-padded buffer of the rank that owns the expert (peer stores);
* ``pull_rows``: it later reads the expert's output row from there while applying the gate weight
  (peer loads, fp32 accumulation).

The two primitives are each other's adjoint, so the backward pass is made of the same two kernels.
Before a layer the ranks exchange their per-expert counts (a few hundred bytes written into every
peer's table) and derive the same row layout from them. Every primitive is bracketed by the
bounded flag barrier of :class:`PeerRuntime`, which is what makes the shared buffers safe to
recycle; all ranks must issue the same sequence of calls.

Copies are avoided where the data has to outlive the exchange anyway: a layer that passes its
``slot`` gets a landing buffer and an outbox of its own. The rows pushed to this rank in the
forward pass are what autograd keeps for the weight gradients, so they stay where they landed; the
down-projection writes the expert outputs straight into the layer's outbox, from where the peers
pull them in the forward pass and again (for the gate-weight gradients) in the backward pass.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor

from ohara_b200.ops._ext import ext
from ohara_b200.parallel.peer import PeerRuntime, SymmetricBuffer

from ohara_b200.ops.moe import TILE  # rows every expert segment is padded to (a GEMM pair tile)
from ohara_b200.utils.checks import debug_checks_enabled, validate_expert_parallel_plan
from ohara_b200.utils.profiling import nvtx_annotate

_DEBUG_CHECKS = debug_checks_enabled()


@dataclass
class DispatchPlan:
    dest_rank: Tensor   # (pairs,) owner rank of each (token, expert) pair
    dest_row: Tensor    # (pairs,) row in the owner's padded buffer, -1 when dropped
    tile_expert: Tensor  # local expert of every TILE-row block of this rank's buffer (-1 unused)
    k_offsets: Tensor   # (local experts + 1,) segment boundaries in this rank's buffer
    fill: Tensor        # (2, local experts) padding rows to clear
    rows_used: Tensor   # (1,) rows the full layout needs on this rank (above capacity = drops)
    top_k: int


class EPWorkspace:
    """Symmetric buffers of one expert-parallel group.

    ``capacity_rows`` (a multiple of 128) bounds the rows any rank may receive for its experts in
    one layer; pairs beyond it are dropped (a capacity factor). ``width`` is the widest row moved
    (the model dimension)."""

    def __init__(self, group, num_experts: int, capacity_rows: int, width: int,
                 wait_limit_s: float = 10.0) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("expert parallelism over peer memory supports up to 8 ranks")
        if num_experts % self.world or capacity_rows % TILE:
            raise ValueError("experts must divide over the ranks and capacity_rows must be a "
                             "multiple of 128")
        self.num_experts = num_experts
        self.local_experts = num_experts // self.world
        self.capacity_rows = capacity_rows
        self.width = width
        self.runtime = PeerRuntime(group, wait_limit_s)
        self.tables = SymmetricBuffer(self.world * num_experts * 4, group)
        self.landing = SymmetricBuffer(capacity_rows * width * 2, group)   # rows pushed to me
        self.outbox = SymmetricBuffer(capacity_rows * width * 2, group)    # rows peers pull from me
        # per-layer buffers (see the module docstring), created at the layer's first forward pass
        self.landing_slots: dict[int, SymmetricBuffer] = {}
        self.outbox_slots: dict[int, SymmetricBuffer] = {}
        self.device = self.tables.device
        torch.cuda.synchronize()
        dist.barrier(group=group)

    # -- layout ------------------------------------------------------------------------------------
    def plan(self, indices: Tensor, counts: Tensor) -> DispatchPlan:
        """Agree on the row layout for int32 ``indices (N, k)`` with per-expert ``counts (E,)``."""
        self.runtime.barrier()  # nobody is still reading the previous table
        ext().ep_publish_counts(self.tables.pointers, counts.contiguous(), self.rank)
        self.runtime.barrier()
        table = self.tables.typed(torch.int32)
        parts = ext().ep_plan(table, indices.contiguous(), self.rank, self.world, TILE,
                              self.capacity_rows)
        plan = DispatchPlan(*parts, top_k=indices.shape[1])
        if _DEBUG_CHECKS:  # OHARA_DEBUG_CHECKS=1: verify the tables on the host (synchronises)
            validate_expert_parallel_plan(
                indices, plan.dest_rank, plan.dest_row, plan.tile_expert, plan.k_offsets,
                world=self.world, num_experts=self.num_experts,
                capacity_rows=self.capacity_rows, tile=TILE)
        return plan

    # -- per-layer buffers -----------------------------------------------------------------------------
    def _slot(self, table: dict[int, SymmetricBuffer], slot: int) -> SymmetricBuffer:
        """The layer's own symmetric buffer; the first request creates it (a collective: every
        rank reaches a layer's first forward pass at the same point of the program)."""
        buffer = table.get(slot)
        if buffer is None:
            buffer = table[slot] = SymmetricBuffer(self.capacity_rows * self.width * 2, self.group)
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        return buffer

    def outbox_rows(self, slot: int, d: int) -> Tensor:
        """This rank's ``(capacity_rows, d)`` outbox of layer ``slot``: the buffer to compute the
        expert outputs into, so that the peers can pull them without a copy."""
        buffer = self._slot(self.outbox_slots, slot)
        return buffer.typed(torch.bfloat16)[: self.capacity_rows * d].view(self.capacity_rows, d)

    def _published(self, padded: Tensor) -> SymmetricBuffer | None:
        """The outbox ``padded`` already lives in, if any."""
        for buffer in self.outbox_slots.values():
            if buffer.local.data_ptr() == padded.data_ptr():
                return buffer
        return None

    # -- data movement -------------------------------------------------------------------------------
    @nvtx_annotate("ep.dispatch")
    def push_rows(self, rows: Tensor, plan: DispatchPlan, scale: Tensor | None = None,
                  slot: int | None = None) -> Tensor:
        """Send row ``t`` of ``rows (N, d)`` to the owners of its ``k`` experts (times ``scale``);
        returns this rank's padded ``(capacity_rows, d)`` buffer of received rows.

        With ``slot`` the rows land in that layer's own buffer and the returned tensor *is* that
        buffer (valid until the layer's next forward pass). Without it they land in the shared
        buffer, which the next push overwrites: the caller must consume the result before it
        issues another exchange (the backward pass does: the gradient rows feed the expert GEMMs
        of the same layer at once)."""
        d = rows.shape[1]
        if slot is None:
            target = self.landing
            self.runtime.barrier()  # every rank has consumed what it received last time
        else:
            # no rank can still be reading this layer's buffer: its last readers ran a whole
            # step ago, and the barriers of ``plan`` lie between them and this push
            target = self._slot(self.landing_slots, slot)
        ext().ep_push_rows(rows.contiguous(), plan.dest_rank, plan.dest_row, scale,
                           target.pointers, plan.top_k, self.capacity_rows)
        self.runtime.barrier()  # all rows have landed
        landed = target.typed(torch.bfloat16)[: self.capacity_rows * d].view(self.capacity_rows, d)
        ext().ep_zero_fill(plan.fill, landed, d, self.capacity_rows)
        return landed

    @nvtx_annotate("ep.combine")
    def pull_rows(self, padded: Tensor, plan: DispatchPlan, scale: Tensor | None = None,
                  other: Tensor | None = None, want_out: bool = True):
        """Adjoint of ``push_rows``: ``out[t] = sum_i scale[t, i] * padded_owner[row(t, i)]`` read
        from the owners' buffers; with ``other (N, d)`` also the per-pair dot products."""
        d = padded.shape[1]
        source = self._published(padded)
        if source is None:  # not in an outbox yet: publish a copy in the shared one
            source = self.outbox
            mine = source.typed(torch.bfloat16)[: self.capacity_rows * d].view(self.capacity_rows, d)
            mine.copy_(padded)
        self.runtime.barrier()  # everyone's rows are published
        out, dots = ext().ep_pull_combine(source.pointers, plan.dest_rank, plan.dest_row, scale,
                                          other, plan.top_k, d, want_out, self.capacity_rows)
        self.runtime.barrier()  # everyone has finished reading before the outbox is reused
        return out, dots


class LazyEPWorkspace:
    """Creates the group's :class:`EPWorkspace` at the first routed batch, when the number of
    (token, expert) pairs per rank is known: ``capacity_rows`` is ``capacity_factor`` times a
    rank's fair share of rows plus the per-expert tile padding. All ranks reach that point
    together (the layers run in lock step)."""

    def __init__(self, group, num_experts: int, width: int, capacity_factor: float = 2.0,
                 wait_limit_s: float = 10.0) -> None:
        self.group, self.num_experts, self.width = group, num_experts, width
        self.capacity_factor, self.wait_limit_s = capacity_factor, wait_limit_s
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.workspace: EPWorkspace | None = None

    def materialize(self, pairs_per_rank: int) -> EPWorkspace:
        if self.workspace is None:
            local = self.num_experts // self.world
            rows = int(self.capacity_factor * pairs_per_rank) + local * TILE
            rows = (rows + TILE - 1) // TILE * TILE
            self.workspace = EPWorkspace(self.group, self.num_experts, rows, self.width,
                                         self.wait_limit_s)
        return self.workspace


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x16: Tensor, plan: DispatchPlan, workspace: EPWorkspace,
                slot: int | None = None) -> Tensor:
        ctx.plan, ctx.workspace = plan, workspace
        landed = workspace.push_rows(x16, plan, slot=slot)
        # without a buffer of its own the layer must keep a copy: the shared landing buffer is
        # overwritten by the next exchange, the rows are needed again for the weight gradients
        return landed if slot is not None else landed.clone()

    @staticmethod
    def backward(ctx, dx_pad: Tensor):
        dx, _ = ctx.workspace.pull_rows(dx_pad.contiguous(), ctx.plan)
        return dx, None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_pad: Tensor, weights: Tensor, plan: DispatchPlan, workspace: EPWorkspace):
        weights = weights.contiguous()
        out, _ = workspace.pull_rows(y_pad, plan, weights.view(-1))
        ctx.save_for_backward(y_pad, weights)
        ctx.plan, ctx.workspace = plan, workspace
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        y_pad, weights = ctx.saved_tensors
        ws, plan = ctx.workspace, ctx.plan
        dout = dout.contiguous()
        # Both exchanges run on every rank whether or not this rank needs the result: the ranks
        # must issue the same sequence of collectives.
        dy_pad = ws.push_rows(dout, plan, weights.view(-1))
        _, dots = ws.pull_rows(y_pad, plan, None, dout, want_out=False)
        return dy_pad, dots.view_as(weights), None, None


def expert_parallel_swiglu(flat_x: Tensor, indices: Tensor, weights: Tensor, counts: Tensor,
                           w_gate: Tensor, w_up: Tensor, w_down: Tensor,
                           workspace: EPWorkspace, slot: int | None = None) -> Tensor:
    """Routed SwiGLU experts with the expert dimension sharded over the group.

    ``indices (N, k)`` are *global* expert ids chosen by this rank's router for its own tokens;
    ``w_gate / w_up (E_local, d, h)`` and ``w_down (E_local, h, d)`` are this rank's experts.
    ``slot`` (a small integer unique to the calling layer) gives the layer its own landing
    buffer and outbox, which removes the copies out of and into the shared ones."""
    from ohara_b200.ops import swiglu
    from ohara_b200.ops.grouped import grouped_linear

    x16 = flat_x if flat_x.dtype == torch.bfloat16 else flat_x.to(torch.bfloat16)
    indices = indices if indices.dtype == torch.int32 else indices.int()
    if isinstance(workspace, LazyEPWorkspace):
        workspace = workspace.materialize(indices.numel())
    plan = workspace.plan(indices, counts)
    x_pad = _DispatchFn.apply(x16.contiguous(), plan, workspace, slot)
    gate = grouped_linear(x_pad, w_gate, plan.tile_expert, plan.k_offsets)
    up = grouped_linear(x_pad, w_up, plan.tile_expert, plan.k_offsets)
    hidden = swiglu(gate, up)
    width = w_down.shape[2]
    out = (lambda: workspace.outbox_rows(slot, width)) if slot is not None else None
    y_pad = grouped_linear(hidden, w_down, plan.tile_expert, plan.k_offsets, out)
    return _CombineFn.apply(y_pad, weights.float(), plan, workspace)
