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
        # recompute the blocks in the backward pass if the model was asked to
        self.activation_checkpointing = bool(getattr(model, "activation_checkpointing", False))

    def hidden(self, x: Tensor) -> Tensor:
        """Hidden states leaving this stage (after the final norm on the last stage)."""
        from ohara_b200 import ops

        h = ops.embedding(x, self.token_emb.weight) if self.is_first else x
        seq = h.size(1)
        if seq > self.config.max_sequence_length:
            raise ValueError("input exceeds max_sequence_length")
        freqs = (self.freq_cos[:seq], self.freq_sin[:seq])
        pending = None  # residual branch output not yet added: fused into the next norm
        recompute = self.activation_checkpointing and self.training and torch.is_grad_enabled()
        for layer in self.layers:
            if recompute:
                from ohara_b200.models.llama import _checkpointed_block

                h, pending = _checkpointed_block(layer, h, pending, freqs)
            else:
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


# --------------------------------------------------------------------------------------------------
# A pipeline stage behind the model interface the trainer and the engine use
# --------------------------------------------------------------------------------------------------
class _PipelineStep(torch.autograd.Function):
    """Forward: the loss of the step (computed by the last stage, made known to every stage).
    Backward: runs the backward pass of every micro-batch of this stage in the order of the
    forward passes, receiving the output gradients from the next stage and sending the input
    gradients to the previous one. The autograd graphs of the micro-batches stay private to the
    stage; what the outside world sees is one scalar whose gradient scales all of them."""

    @staticmethod
    def forward(ctx, anchor: Tensor, owner: "PipelinedLlama", saved: list, loss_value: Tensor):
        ctx.owner, ctx.saved = owner, saved
        return loss_value.clone()

    @staticmethod
    def backward(ctx, grad_out: Tensor):
        owner: PipelinedLlama = ctx.owner
        for stage_input, output in ctx.saved:
            if owner.is_last:
                torch.autograd.backward(output, grad_out.to(output.dtype))
            else:
                grad = torch.empty_like(output)
                dist.recv(grad, owner._peer(+1), group=owner.group)
                # the gradient arrives already scaled by the last stage
                torch.autograd.backward(output, grad)
            if not owner.is_first:
                owner._send(stage_input.grad, -1)
        owner._drain()
        ctx.saved = None
        return None, None, None, None


class PipelinedLlama(nn.Module):
    """One pipeline stage of a Llama that looks like the whole model to its caller.

    ``model(tokens, targets=...)`` splits the batch into micro-batches, runs this stage's forward
    pass for each of them (activations travel to the next rank with point-to-point sends) and
    returns the summed cross-entropy of the step on *every* stage; calling ``backward()`` on it
    (times any scale) runs the backward passes of all micro-batches and leaves the gradients on
    this stage's parameters. ``model(tokens)`` without targets returns the logits on every
    stage (evaluation). This is the all-forward-then-all-backward (GPipe) schedule: the trainer's
    contract "forward returns a loss, the engine calls backward on it" leaves no room to interleave
    the two; :class:`PipelineRunner` offers 1F1B to callers that drive the schedule themselves.

    The ranks of a pipeline must be fed the same batches (the engine's data-parallel rank does
    not depend on the pipeline coordinate)."""

    supports_fused_loss = True
    pipeline_stage = True  # optimizer builders: the embedding or the head may live elsewhere

    # the parts of the model this stage holds, under the names the optimizer builders look for
    @property
    def token_emb(self):
        return self.stage.token_emb

    @property
    def vocab_proj(self):
        return self.stage.vocab_proj

    @property
    def layers(self):
        return self.stage.layers

    def __init__(self, stage: LlamaStage, group=None, micro_batch_size: int = 1) -> None:
        super().__init__()
        self.stage = stage
        self.group = group
        self.micro_batch_size = max(1, int(micro_batch_size))
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.is_first, self.is_last = self.rank == 0, self.rank == self.world - 1
        self.config = stage.config
        self._pending: deque = deque()

    # -- point-to-point plumbing ----------------------------------------------------------------
    def _peer(self, offset: int) -> int:
        target = self.rank + offset
        return dist.get_global_rank(self.group, target) if self.group is not None else target

    def _send(self, tensor: Tensor, offset: int) -> None:
        tensor = tensor.contiguous()
        self._pending.append((dist.isend(tensor, self._peer(offset), group=self.group), tensor))
        while len(self._pending) > 4 * self.world:
            self._pending.popleft()[0].wait()

    def _drain(self) -> None:
        while self._pending:
            self._pending.popleft()[0].wait()

    def _activation_dtype(self, reference: Tensor) -> torch.dtype:
        if reference.is_cuda and torch.is_autocast_enabled("cuda"):
            return torch.get_autocast_dtype("cuda")
        return next(self.stage.parameters()).dtype

    def _stage_forward(self, tokens: Tensor) -> tuple[Tensor, Tensor]:
        """(input of this stage that needs a gradient or the tokens, hidden states leaving it)."""
        if self.is_first:
            stage_input = tokens
        else:
            shape = (tokens.shape[0], tokens.shape[1], self.config.hidden_size)
            stage_input = torch.empty(shape, device=tokens.device,
                                      dtype=self._activation_dtype(tokens))
            dist.recv(stage_input, self._peer(-1), group=self.group)
            stage_input.requires_grad_(torch.is_grad_enabled())
        return stage_input, self.stage.hidden(stage_input)

    # -- the model interface -------------------------------------------------------------------
    def forward(self, x: Tensor, kv_cache=None, position_ids=None, *, targets: Tensor | None = None,
                ignore_index: int = -1, loss_scale: Tensor | float | None = None) -> Tensor:
        if kv_cache is not None:
            raise NotImplementedError("cached decoding runs on an unsplit model")
        if targets is None:
            return self._logits(x)
        from ohara_b200 import ops

        micro = min(self.micro_batch_size, x.shape[0])
        saved: list[tuple[Tensor, Tensor]] = []
        total = torch.zeros((), device=x.device, dtype=torch.float32)
        for tokens, labels in zip(x.split(micro), targets.split(micro)):
            stage_input, hidden = self._stage_forward(tokens)
            if self.is_last:
                loss = ops.linear_cross_entropy(hidden, self.stage.vocab_proj.weight, labels,
                                                ignore_index, loss_scale)
                total = total + loss.detach().float()
                saved.append((stage_input, loss))
            else:
                self._send(hidden.detach(), +1)
                saved.append((stage_input, hidden))
        self._drain()
        # every stage reports the loss of the step
        dist.broadcast(total, src=self._peer(self.world - 1 - self.rank), group=self.group)
        if not torch.is_grad_enabled():
            return total
        anchor = torch.zeros((), device=x.device, requires_grad=True)
        return _PipelineStep.apply(anchor, self, saved, total)

    @torch.no_grad()
    def _logits(self, x: Tensor) -> Tensor:
        micro = min(self.micro_batch_size, x.shape[0])
        pieces = []
        for tokens in x.split(micro):
            _, hidden = self._stage_forward(tokens)
            if self.is_last:
                pieces.append(self.stage.vocab_proj(hidden).float())
            else:
                self._send(hidden, +1)
        self._drain()
        shape = (x.shape[0], x.shape[1], self.config.vocab_size)
        logits = torch.cat(pieces) if self.is_last else torch.empty(shape, device=x.device)
        dist.broadcast(logits, src=self._peer(self.world - 1 - self.rank), group=self.group)
        return logits

    def estimate_flops(self, sequence_length: int | None = None) -> float:
        """Forward + backward FLOPs per token of the *whole* model (every stage reports the same
        figure, so throughput lines agree across ranks)."""
        return float(getattr(self, "_model_flops", 0.0))
