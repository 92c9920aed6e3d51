"""Pipeline-parallel schedules: GPipe and 1F1B over point-to-point sends.

The reference ships only the plan dataclasses (ohara/runtime/pipeline.py:8-32: no stage split, no
schedule, no send / recv); this is the missing executor. A rank owns one stage module; activations
flow to the next rank and their gradients back with c10d point-to-point operations (NCCL on GPUs,
gloo on CPU) - pipeline traffic is one activation tensor per micro-batch per boundary, which the
library path handles well, so no custom kernel is involved.

``PipelineRunner.step(micro_inputs, micro_targets)`` runs one optimisation step's worth of
micro-batches and leaves gradients on the stage's parameters:

* ``GPIPE``: all forwards, then all backwards (activations of every micro-batch are alive).
* ``ONE_FWD_ONE_BWD``: ``world - rank - 1`` warm-up forwards, then alternate one forward and one
  backward, then drain; at most ``world - rank`` activations are alive on a rank.

Sends are non-blocking (the handle is awaited before its buffer can be reused or freed), receives
blocking: neighbouring ranks that want to send to each other at the same time cannot deadlock.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Callable, Sequence

import torch
import torch.distributed as dist
from torch import Tensor, nn

from ohara_b200.runtime.enums import PipelineScheduleType


class PipelineRunner:
    """Executes ``stage`` as rank ``dist.get_rank(group)`` of a linear pipeline.

    ``loss_fn(output, target) -> scalar`` is used by the last stage only. The first stage receives
    its inputs from ``step``; every other stage needs ``activation_shape`` / ``activation_dtype``
    (shape of one micro-batch of its input) to allocate receive buffers.
    """

    def __init__(self, stage: nn.Module, loss_fn: Callable[[Tensor, Tensor], Tensor] | None = None, *,
                 group=None, schedule: PipelineScheduleType = PipelineScheduleType.ONE_FWD_ONE_BWD,
                 activation_shape: Sequence[int] | None = None,
                 activation_dtype: torch.dtype = torch.float32,
                 device: torch.device | str | None = None) -> None:
        self.stage, self.loss_fn, self.group = stage, loss_fn, group
        self.schedule = PipelineScheduleType(schedule)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        if self.last and loss_fn is None:
            raise ValueError("the last pipeline stage needs a loss function")
        if not self.first and activation_shape is None:
            raise ValueError("stages after the first need the shape of their input micro-batch")
        self.activation_shape = tuple(activation_shape) if activation_shape is not None else None
        self.activation_dtype = activation_dtype
        self.device = torch.device(device) if device is not None else next(
            stage.parameters()).device
        self._pending: deque = deque()  # (work handle, tensor kept alive)

    # -- neighbours ------------------------------------------------------------------------------
    def _peer(self, offset: int) -> int:
        target = self.rank + offset
        return dist.get_global_rank(self.group, target) if self.group is not None else target

    def _send(self, tensor: Tensor, offset: int) -> None:
        tensor = tensor.contiguous()
        self._pending.append((dist.isend(tensor, self._peer(offset), group=self.group), tensor))
        while len(self._pending) > 2 * self.world:  # bound the number of buffers kept alive
            self._pending.popleft()[0].wait()

    def _recv(self, offset: int) -> Tensor:
        buffer = torch.empty(self.activation_shape, dtype=self.activation_dtype, device=self.device)
        dist.recv(buffer, self._peer(offset), group=self.group)
        return buffer

    # -- one micro-batch --------------------------------------------------------------------------
    def _forward(self, micro_input: Tensor | None, target: Tensor | None):
        if self.first:
            stage_input = micro_input
        else:
            stage_input = self._recv(-1).requires_grad_()
        output = self.stage(stage_input)
        if self.last:
            loss = self.loss_fn(output, target)
            return stage_input, loss
        self._send(output.detach(), +1)
        return stage_input, output

    def _backward(self, stage_input: Tensor, output: Tensor, scale: float) -> None:
        if self.last:
            (output * scale).backward()
        else:
            grad = torch.empty_like(output)
            dist.recv(grad, self._peer(+1), group=self.group)
            output.backward(grad)
        if not self.first:
            self._send(stage_input.grad, -1)

    # -- one step ----------------------------------------------------------------------------------
    def step(self, micro_inputs: Sequence[Tensor] | None, micro_targets: Sequence[Tensor] | None,
             num_micro_batches: int | None = None) -> Tensor | None:
        """Run all micro-batches (forward and backward). The last stage returns the mean loss,
        the others ``None``. ``micro_inputs`` is read on the first stage, ``micro_targets`` on the
        last; the other argument may be ``None`` there, with ``num_micro_batches`` given."""
        count = num_micro_batches or len(micro_inputs if micro_inputs is not None else micro_targets)
        scale = 1.0 / count
        get_in = (lambda i: micro_inputs[i]) if self.first else (lambda i: None)
        get_tg = (lambda i: micro_targets[i]) if self.last else (lambda i: None)
        saved: deque = deque()
        losses: list[Tensor] = []

        def forward(i: int) -> None:
            stage_input, output = self._forward(get_in(i), get_tg(i))
            if self.last:
                losses.append(output.detach())
            saved.append((stage_input, output))

        def backward() -> None:
            stage_input, output = saved.popleft()
            self._backward(stage_input, output, scale)

        if self.schedule == PipelineScheduleType.GPIPE:
            for i in range(count):
                forward(i)
            for _ in range(count):
                backward()
        else:
            warmup = min(self.world - self.rank - 1, count)
            for i in range(warmup):
                forward(i)
            for i in range(warmup, count):
                forward(i)
                backward()
            for _ in range(warmup):
                backward()
        while self._pending:
            self._pending.popleft()[0].wait()
        if self.last:
            return torch.stack(losses).mean()
        return None


def split_sequential(layers: Sequence[nn.Module], world: int, rank: int) -> nn.Sequential:
    """Contiguous, balanced slice of ``layers`` for pipeline rank ``rank`` (earlier ranks take the
    remainder, like ``torch.chunk``)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad pipeline rank / world")
    if len(layers) < world:
        raise ValueError("fewer layers than pipeline stages")
    base, extra = divmod(len(layers), world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return nn.Sequential(*layers[begin:end])
