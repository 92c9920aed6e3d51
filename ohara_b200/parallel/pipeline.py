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


def stage_bounds(num_layers: int, world: int, rank: int) -> tuple[int, int]:
    """``[begin, end)`` of the transformer blocks owned by pipeline rank ``rank`` (the same
    contiguous, balanced split as :func:`split_sequential`)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad pipeline rank / world")
    if num_layers < world:
        raise ValueError("fewer layers than pipeline stages")
    base, extra = divmod(num_layers, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class LlamaStage(nn.Module):
    """One pipeline stage of a :class:`ohara_b200.models.llama.Llama`.

    The stage keeps only its own sub-modules of ``model``: the token embedding on the first rank,
    a contiguous run of transformer blocks, the final norm and the output projection on the last
    rank (plus the rotary tables, which every stage needs). The first stage maps token ids
    ``(B, T)`` to hidden states, the others map hidden states to hidden states, and the last one
    returns logits - or, given ``targets``, the summed cross-entropy through the fused
    projection + loss kernel, so that no logits tensor is materialised:

        stage = LlamaStage(Llama(cfg), world, rank)
        runner = PipelineRunner(stage, loss_fn=stage.loss, activation_shape=(B, T, hidden), ...)

    Tied input / output embeddings would live on two different ranks and are rejected.
    """

    def __init__(self, model: nn.Module, world: int, rank: int) -> None:
        super().__init__()
        cfg = model.config
        if world > 1 and model.vocab_proj.weight is model.token_emb.weight:
            raise ValueError("pipeline stages cannot share tied embeddings: use weight_tying=False")
        begin, end = stage_bounds(len(model.layers), world, rank)
        self.config = cfg
        self.is_first, self.is_last = rank == 0, rank == world - 1
        self.layer_range = (begin, end)
        self.token_emb = model.token_emb if self.is_first else None
        self.layers = nn.ModuleList(list(model.layers)[begin:end])
        self.norm = model.norm if self.is_last else None
        self.vocab_proj = model.vocab_proj if self.is_last else None
        self.register_buffer("freq_cos", model.freq_cos, persistent=False)
        self.register_buffer("freq_sin", model.freq_sin, persistent=False)

    def hidden(self, x: Tensor) -> Tensor:
        """Hidden states leaving this stage (after the final norm on the last stage)."""
        from ohara_b200 import ops

        h = ops.embedding(x, self.token_emb.weight) if self.is_first else x
        seq = h.size(1)
        if seq > self.config.max_sequence_length:
            raise ValueError("input exceeds max_sequence_length")
        freqs = (self.freq_cos[:seq], self.freq_sin[:seq])
        pending = None  # residual branch output not yet added: fused into the next norm
        for layer in self.layers:
            h, pending = layer.forward_deferred(h, pending, freqs, None, None)
        if self.is_last:
            return ops.add_rms_norm(h, pending, self.norm.weight, self.norm.eps)[0]
        return h if pending is None else h + pending

    def forward(self, x: Tensor) -> Tensor:
        h = self.hidden(x)
        return self.vocab_proj(h) if self.is_last else h

    def loss(self, logits: Tensor, targets: Tensor, ignore_index: int = -1) -> Tensor:
        """Mean cross-entropy of the last stage's logits (``loss_fn`` of the runner)."""
        return torch.nn.functional.cross_entropy(
            logits.float().reshape(-1, logits.size(-1)), targets.reshape(-1),
            ignore_index=ignore_index)
