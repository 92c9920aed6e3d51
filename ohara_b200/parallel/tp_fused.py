"""Tensor-parallel linears whose collectives run *inside* the tcgen05 GEMM over NVLink peer memory.

Sequence-parallel Megatron-style layers need two patterns, both provided here as autograd ops:

* ``column_parallel_fused``: ``y = all_gather(x_local) @ W_shard^T``. The local rows are copied into
  a symmetric staging buffer and a flag is published; the copy engines pull the peers' rows while
  the GEMM is already multiplying its own rows, and the GEMM's TMA producer waits on a per-block
  "arrived" flag just before it first needs a remote block. The backward is
  ``dx_local = reduce_scatter(dy @ W_shard)`` through the other pattern.
* ``row_parallel_fused``: ``y_local = reduce_scatter(x @ W_shard^T)``. The GEMM epilogue stores each
  row block of the partial product directly into the owner's receive slot for this rank (16-byte
  peer stores from the accumulator registers), remote blocks first; after a flag exchange a small
  kernel on the owner sums the slots. The backward is the first pattern.

Weight gradients need the gathered operand itself; it is the buffer the copies landed in, so no
second collective is issued.

Buffers are double-buffered per pattern and recycled under one rule: every staged tensor is
consumed by a kernel that waits for *all* peers' flags of that epoch, so a rank can be at most one
fused op ahead of its slowest peer and never overwrites a buffer that is still being read. All
ranks of the group must issue the same sequence of fused ops. Waits are bounded
(``wait_limit_s``); a timeout surfaces through ``ops.check_status()``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ohara_b200.ops._ext import ext
from ohara_b200.parallel.peer import SymmetricBuffer, release_stream_waits
from ohara_b200.utils.profiling import nvtx_annotate

_AG_SLOT = 0   # flag slots [0, world): "my staged rows for epoch e are complete"
_RS_SLOT = 16  # flag slots [16, 16 + world): "my pushes for epoch e are complete"


class StagedRows:
    """Rows staged for an all-gather: workspace buffer index, epoch, shape and the events that
    mark the arrival of every peer's rows in the local gathered buffer."""

    __slots__ = ("buffer", "epoch", "rows", "width", "arrived")

    def __init__(self, buffer: int, epoch: int, rows: int, width: int, arrived) -> None:
        self.buffer, self.epoch, self.rows, self.width, self.arrived = buffer, epoch, rows, width, arrived


class TPWorkspace:
    """Symmetric staging / receive buffers and flags of one tensor-parallel group.

    ``rows_local`` x ``width`` bf16 elements bound the largest per-rank activation block that the
    fused ops will see (``rows_local`` must be a multiple of 128, the GEMM tile height).

    All-gather side: each rank copies its rows into a symmetric staging buffer and publishes a
    flag. A side stream then pulls every peer's rows into a local gathered buffer with the copy
    engines (no SM is used): a stream-ordered wait on the peer's flag, the peer-to-peer copy, and a
    stream-ordered write of a local "arrived" flag. The GEMM on the main stream multiplies its own
    rows first and waits (bounded, in the TMA producer) on the arrived flag of each remote block
    just before it needs it, so the transfers overlap the math and every remote row crosses NVLink
    exactly once however many column tiles re-read it.
    """

    def __init__(self, group, rows_local: int, width: int, wait_limit_s: float = 10.0) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("fused tensor parallelism supports up to 8 ranks")
        self.capacity = rows_local * width
        self.wait_limit_s = wait_limit_s
        self.flags = SymmetricBuffer(4096, group)
        self.gather = [SymmetricBuffer(self.capacity * 2, group) for _ in range(2)]
        self.receive = [SymmetricBuffer(self.capacity * 2 * self.world, group) for _ in range(2)]
        self.device = self.flags.device
        self.gathered = [torch.empty(self.world * self.capacity, device=self.device,
                                     dtype=torch.bfloat16) for _ in range(2)]
        self.arrived_flags = torch.zeros(64, device=self.device, dtype=torch.int32)
        # Several copy streams so that the pulls from different peers overlap instead of queueing
        # behind each other's flag waits.
        self.copy_streams = [torch.cuda.Stream(device=self.device, priority=-1)
                             for _ in range(max(1, min(self.world - 1, 4)))]
        self.gather_epoch = 0
        self.scatter_epoch = 0
        self.poisoned = False
        self._maps: dict[tuple[int, int, int], Tensor] = {}
        torch.cuda.synchronize()
        dist.barrier(group=group)  # every rank has opened every buffer before the first signal

    def abort(self) -> None:
        """Release the copy streams: satisfy every stream-ordered wait this workspace may have
        queued on a peer's "staged" flag (they live in this rank's flag buffer) and mark the
        workspace unusable. The kernels' own waits are bounded and have already returned with a
        status; only the copy engines' waits need this way out. Called by the engine when a
        collective timed out, a peer was reported lost or the step watchdog fired."""
        self.poisoned = True
        release_stream_waits([self._flag_address(_AG_SLOT + r) for r in range(self.world)],
                             self.device)

    def _flag_address(self, slot: int) -> int:
        return self.flags.pointers[self.rank] + 4 * slot

    def _gathered_blocks(self, index: int, rows: int, width: int) -> Tensor:
        return self.gathered[index][: self.world * rows * width].view(self.world, rows, width)

    # -- all-gather side ----------------------------------------------------------------------------
    @nvtx_annotate("tp.stage_rows")
    def stage(self, x_local: Tensor) -> StagedRows:
        rows, width = x_local.shape
        if self.poisoned:
            raise RuntimeError("this tensor-parallel workspace was aborted after a lost peer or a "
                               "timed-out collective; rebuild the engine to continue")
        if rows % 128 or rows * width > self.capacity:
            raise ValueError(f"cannot stage a {rows} x {width} block (rows must be a multiple of 128 "
                             f"and fit {self.capacity} elements)")
        self.gather_epoch += 1
        epoch, index = self.gather_epoch, self.gather_epoch % 2
        mine = self.gather[index].typed(torch.bfloat16)[: rows * width].view(rows, width)
        mine.copy_(x_local)
        ext().tp_signal(self.flags.pointers, _AG_SLOT, self.rank, epoch)
        main = torch.cuda.current_stream(self.device)
        staged_event = torch.cuda.Event()
        staged_event.record(main)
        # The side stream may touch the gathered buffer only after everything already queued on
        # the main stream (the previous readers of this buffer) has finished.
        blocks = self._gathered_blocks(index, rows, width)
        arrived = []
        for lane, stream in enumerate(self.copy_streams):
            stream.wait_event(staged_event)
            with torch.cuda.stream(stream):
                for hop in range(1 + lane, self.world, len(self.copy_streams)):
                    src = (self.rank + hop) % self.world
                    ext().stream_wait_value32(self._flag_address(_AG_SLOT + src), epoch)
                    remote = self.gather[index].typed(torch.bfloat16, rank=src)[: rows * width]
                    blocks[src].copy_(remote.view(rows, width))
                    ext().stream_write_value32(self.arrived_flags.data_ptr() + 4 * src, epoch)
                if lane == 0:
                    blocks[self.rank].copy_(mine)  # completes the gathered tensor (weight gradients)
                event = torch.cuda.Event()
                event.record(stream)
                arrived.append(event)
        return StagedRows(index, epoch, rows, width, arrived)

    @nvtx_annotate("tp.all_gather_gemm")
    def gemm_from(self, staged: StagedRows, weight16: Tensor, b_mn: bool, out_features: int) -> Tensor:
        """``all_gather(staged) @ op(weight16)``: ``(world * rows, out_features)`` bf16."""
        key = (staged.buffer, staged.rows, staged.width)
        maps = self._maps.get(key)
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        local = self.gather[staged.buffer].typed(torch.bfloat16)[: staged.rows * staged.width]
        local = local.view(staged.rows, staged.width)
        if maps is None:
            blocks = self._gathered_blocks(staged.buffer, staged.rows, staged.width)
            # own rows straight from the staging buffer, remote rows from where the copies land
            bases = [local.data_ptr() if r == self.rank else blocks[r].data_ptr()
                     for r in range(self.world)]
            maps = ext().peer_row_maps(bases, staged.rows, staged.width, staged.width, index)
            self._maps[key] = maps
        out = torch.empty(staged.rows * self.world, out_features, device=local.device,
                          dtype=torch.bfloat16)
        ext().gemm_gather_a(maps, local, weight16, out, b_mn, self.arrived_flags.data_ptr(),
                            staged.epoch, self.rank, self.world, self.wait_limit_s)
        return out

    @nvtx_annotate("tp.all_gather")
    def gather_from(self, staged: StagedRows) -> Tensor:
        """The gathered ``(world * rows, width)`` tensor itself (operand of a weight gradient).
        It aliases a workspace buffer that is recycled two stagings later: consume it at once."""
        for event in staged.arrived:
            torch.cuda.current_stream(self.device).wait_event(event)
        blocks = self._gathered_blocks(staged.buffer, staged.rows, staged.width)
        return blocks.view(self.world * staged.rows, staged.width)

    # -- reduce-scatter side ------------------------------------------------------------------------
    @nvtx_annotate("tp.gemm_reduce_scatter")
    def gemm_reduce_scatter(self, a16: Tensor, weight16: Tensor, b_mn: bool, out_features: int,
                            residual: Tensor | None = None) -> Tensor:
        """``reduce_scatter(a16 @ op(weight16))`` over row blocks: ``(rows / world, out_features)``."""
        rows = a16.shape[0]
        if rows % (128 * self.world):
            raise ValueError("rows per rank must be a multiple of 128")
        rows_local = rows // self.world
        if rows_local * out_features > self.capacity:
            raise ValueError("reduce-scatter block exceeds the workspace")
        self.scatter_epoch += 1
        buffer = self.receive[self.scatter_epoch % 2]
        slot_bytes = rows_local * out_features * 2
        # Row block r goes to rank r's buffer, into the slot that rank keeps for this rank.
        destinations = [buffer.pointers[r] + self.rank * slot_bytes for r in range(self.world)]
        ext().gemm_push_c(a16, weight16, b_mn, destinations, out_features, out_features, self.rank)
        ext().tp_signal(self.flags.pointers, _RS_SLOT, self.rank, self.scatter_epoch)
        slots = buffer.typed(torch.bfloat16)[: self.world * rows_local * out_features]
        slots = slots.view(self.world, rows_local, out_features)
        return ext().tp_reduce_slots(slots, self._flag_address(_RS_SLOT), residual,
                                     self.scatter_epoch, self.wait_limit_s)


class LazyTPWorkspace:
    """Creates the group's :class:`TPWorkspace` at the first fused call, when the per-rank token
    count is known. Every rank reaches that call at the same point of the same step (the layers
    run in lock step), so the collective buffer set-up inside is safe."""

    def __init__(self, group, width: int, wait_limit_s: float = 10.0) -> None:
        self.group, self.width, self.wait_limit_s = group, width, wait_limit_s
        self.workspace: TPWorkspace | None = None

    def materialize(self, rows_local: int) -> TPWorkspace:
        if self.workspace is None:
            self.workspace = TPWorkspace(self.group, rows_local, self.width, self.wait_limit_s)
        return self.workspace


def _bf16(t: Tensor) -> Tensor:
    t = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
    return t.contiguous()


class _ColumnParallelFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local: Tensor, weight: Tensor, workspace: TPWorkspace) -> Tensor:
        from ohara_b200.ops import bf16_weight

        x16 = _bf16(x_local)
        staged = workspace.stage(x16)
        out = workspace.gemm_from(staged, bf16_weight(weight), False, weight.shape[0])
        ctx.save_for_backward(x16, weight)
        ctx.workspace = workspace
        ctx.x_dtype = x_local.dtype
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        from ohara_b200.ops import bf16_weight, matmul_tn

        x16, weight = ctx.saved_tensors
        ws = ctx.workspace
        dy16 = _bf16(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx_local = reduce_scatter(dy @ W): W stored (out_local, in) is the MN-major B here.
            dx = ws.gemm_reduce_scatter(dy16, bf16_weight(weight), True, weight.shape[1])
            dx = dx.to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            gathered = ws.gather_from(ws.stage(x16))
            dw = matmul_tn(dy16, gathered).to(weight.dtype)
        return dx, dw, None


class _ColumnParallelFusedCat(torch.autograd.Function):
    """``all_gather(x_local) @ concat(weight shards).T`` for several column-parallel layers that
    share an input (query | key | value; gate | up): ONE staging of the rows and one gather instead
    of one per layer, one GEMM, and in the backward pass one GEMM -> reduce-scatter for the input
    gradient and one re-gather for all the weight gradients."""

    @staticmethod
    def forward(ctx, x_local: Tensor, workspace: TPWorkspace, *weights: Tensor) -> Tensor:
        from ohara_b200.ops import fused_bf16_weight

        x16 = _bf16(x_local)
        staged = workspace.stage(x16)
        w_cat = fused_bf16_weight(weights)
        out = workspace.gemm_from(staged, w_cat, False, w_cat.shape[0])
        ctx.save_for_backward(x16, *weights)
        ctx.workspace = workspace
        ctx.x_dtype = x_local.dtype
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        from ohara_b200.ops import fused_bf16_weight, matmul_tn

        x16, *weights = ctx.saved_tensors
        ws = ctx.workspace
        dy16 = _bf16(dy)
        dx = None
        grads: list[Tensor | None] = [None] * len(weights)
        if ctx.needs_input_grad[0]:
            w_cat = fused_bf16_weight(weights)  # (sum of out_local, in): MN-major B of dy @ W
            dx = ws.gemm_reduce_scatter(dy16, w_cat, True, w_cat.shape[1]).to(ctx.x_dtype)
        if any(ctx.needs_input_grad[2:]):
            gathered = ws.gather_from(ws.stage(x16))
            dw = matmul_tn(dy16, gathered)
            begin = 0
            for i, weight in enumerate(weights):
                end = begin + weight.shape[0]
                if ctx.needs_input_grad[2 + i]:
                    grads[i] = dw[begin:end].to(weight.dtype)
                begin = end
        return (dx, None, *grads)


class _RowParallelFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, workspace: TPWorkspace) -> Tensor:
        from ohara_b200.ops import bf16_weight

        x16 = _bf16(x)
        out = workspace.gemm_reduce_scatter(x16, bf16_weight(weight), False, weight.shape[0])
        ctx.save_for_backward(x16, weight)
        ctx.workspace = workspace
        ctx.x_dtype = x.dtype
        return out

    @staticmethod
    def backward(ctx, dy_local: Tensor):
        from ohara_b200.ops import bf16_weight, matmul_tn

        x16, weight = ctx.saved_tensors
        ws = ctx.workspace
        staged = ws.stage(_bf16(dy_local))
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx = all_gather(dy) @ W: W stored (out, in_local) is the MN-major B here.
            dx = ws.gemm_from(staged, bf16_weight(weight), True, weight.shape[1]).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = matmul_tn(ws.gather_from(staged), x16).to(weight.dtype)
        return dx, dw, None


def column_parallel_fused(x_local: Tensor, weight: Tensor, workspace: TPWorkspace) -> Tensor:
    """``all_gather(x_local) @ weight.T`` for 2-D ``x_local (rows_local, in)`` and a weight shard
    ``(out_local, in)``; returns ``(world * rows_local, out_local)`` bf16."""
    return _ColumnParallelFused.apply(x_local, weight, workspace)


def column_parallel_fused_cat(x_local: Tensor, weights, workspace: TPWorkspace) -> Tensor:
    """``all_gather(x_local) @ concat(weights).T`` for weight shards ``(out_local_i, in)`` that
    share the input; returns ``(world * rows_local, sum of out_local_i)`` bf16."""
    return _ColumnParallelFusedCat.apply(x_local, workspace, *weights)


def row_parallel_fused(x: Tensor, weight: Tensor, workspace: TPWorkspace) -> Tensor:
    """``reduce_scatter(x @ weight.T)`` for 2-D ``x (rows, in_local)`` and a weight shard
    ``(out, in_local)``; returns this rank's ``(rows / world, out)`` bf16 block."""
    return _RowParallelFused.apply(x, weight, workspace)


def fused_supported(rows_local: int, in_features: int, out_features: int) -> bool:
    return rows_local % 128 == 0 and in_features % 8 == 0 and out_features % 8 == 0
