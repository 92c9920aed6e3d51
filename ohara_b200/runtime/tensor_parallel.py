"""Tensor-parallel plan and the sharded linear layers that implement it.

The plan object and ``llama_default`` rules match the reference (ohara/runtime/tensor_parallel.py:
14-90): fnmatch patterns mapping module names to COLWISE / ROWWISE. The implementation does not use
DTensor: matched ``nn.Linear`` modules are replaced in place by :class:`ColumnParallelLinear` /
:class:`RowParallelLinear`, which keep the local weight shard under the same state-dict key and
place the collectives explicitly (identity/all-reduce pairs, or, when ``sequence_parallel`` is on,
all-gather/reduce-scatter pairs over token blocks: between the parallel regions every rank keeps
``B / tp`` whole sequences, along dim 0, in the fused peer-memory form and in the process-group
form alike). Attention derives its local head count
from the projection width, so query and KV heads are split across ranks (GQA included).
"""

from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from .enums import TensorParallelStyle


@dataclass
class TensorParallelRule:
    module_pattern: str
    style: TensorParallelStyle


@dataclass
class TensorParallelPlan:
    degree: int = 1
    sequence_parallel: bool = False
    rules: list[TensorParallelRule] = field(default_factory=list)

    def validate(self, hidden_size: int | None = None) -> None:
        if self.degree < 1:
            raise ValueError("tensor parallel degree must be >= 1")
        if hidden_size is not None and hidden_size % self.degree != 0:
            raise ValueError(
                f"hidden_size={hidden_size} must be divisible by tensor parallel degree={self.degree}"
            )

    @classmethod
    def llama_default(cls, degree: int, sequence_parallel: bool = False) -> "TensorParallelPlan":
        col, row = TensorParallelStyle.COLWISE, TensorParallelStyle.ROWWISE
        return cls(
            degree=degree,
            sequence_parallel=sequence_parallel,
            rules=[
                TensorParallelRule("layers.*.attn.query", col),
                TensorParallelRule("layers.*.attn.key", col),
                TensorParallelRule("layers.*.attn.value", col),
                TensorParallelRule("layers.*.attn.proj", row),
                TensorParallelRule("layers.*.ff.up", col),
                TensorParallelRule("layers.*.ff.gate", col),
                TensorParallelRule("layers.*.ff.down", row),
            ],
        )

    @classmethod
    def mlp_and_head(cls, degree: int) -> "TensorParallelPlan":
        """Shard only the feed-forward layers and the output head; attention stays replicated.
        For models whose head count the degree does not divide (a 6-head model on 8 ranks):
        the SwiGLU width and the vocabulary still split evenly, and they hold most of the
        weights a decode step has to stream."""
        col, row = TensorParallelStyle.COLWISE, TensorParallelStyle.ROWWISE
        return cls(
            degree=degree,
            sequence_parallel=False,
            rules=[
                TensorParallelRule("layers.*.ff.up", col),
                TensorParallelRule("layers.*.ff.gate", col),
                TensorParallelRule("layers.*.ff.down", row),
                TensorParallelRule("vocab_proj", TensorParallelStyle.COLWISE_GATHERED),
            ],
        )

    def style_for(self, module_fqn: str) -> TensorParallelStyle | None:
        for rule in self.rules:
            if fnmatch.fnmatch(module_fqn, rule.module_pattern):
                return rule.style
        return None


# --------------------------------------------------------------------------------------------------
# Collective autograd pairs
# --------------------------------------------------------------------------------------------------
class _CopyToGroup(torch.autograd.Function):
    """Identity forward, all-reduce(sum) backward: entry of a column-parallel region."""

    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, grad: Tensor):
        grad = grad.contiguous()
        dist.all_reduce(grad, group=ctx.group)
        return grad, None


class _ReduceFromGroup(torch.autograd.Function):
    """All-reduce(sum) forward, identity backward: exit of a row-parallel region."""

    @staticmethod
    def forward(ctx, x: Tensor, group, runtime=None):
        x = x.contiguous()
        if runtime is not None and x.is_cuda:
            # Small messages (decode steps) go through the peer-memory one-shot kernel, larger
            # ones fall through to the c10d collective inside it.
            return runtime.all_reduce_(x)
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, grad: Tensor):
        return grad, None, None


class _GatherFeatures(torch.autograd.Function):
    """All-gather along the last dimension forward, own slice backward (gathered column-parallel
    output)."""

    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        world = dist.get_world_size(group)
        ctx.rank, ctx.width = dist.get_rank(group), x.shape[-1]
        x = x.contiguous()
        if x.is_cuda:  # one collective into one buffer: also what a CUDA-graph capture wants
            stacked = torch.empty((world, *x.shape), device=x.device, dtype=x.dtype)
            dist.all_gather_into_tensor(stacked, x, group=group)
            return stacked.movedim(0, -2).reshape(*x.shape[:-1], world * x.shape[-1])
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x, group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, grad: Tensor):
        begin = ctx.rank * ctx.width
        return grad[..., begin:begin + ctx.width].contiguous(), None


def _reduce_scatter_blocks(x: Tensor, group) -> Tensor:
    """Sum ``x`` over the group and keep this rank's block of dim 0 (gloo has no reduce-scatter:
    there it is an all-reduce and a slice)."""
    world = dist.get_world_size(group)
    chunks = [c.contiguous() for c in x.chunk(world, dim=0)]
    if dist.get_backend(group) == "gloo":
        summed = x.contiguous().clone()
        dist.all_reduce(summed, group=group)
        return summed.chunk(world, dim=0)[dist.get_rank(group)].contiguous()
    out = torch.empty_like(chunks[0])
    dist.reduce_scatter(out, chunks, group=group)
    return out


def _gather_blocks(x: Tensor, group) -> Tensor:
    world = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=0)


class _GatherSequence(torch.autograd.Function):
    """Sequence-parallel entry over the process group: all-gather the ranks' token blocks along
    dim 0 forward, reduce-scatter backward. The blocks are whole sequences (``B / tp`` of them per
    rank), the same layout as the fused gather-GEMM, so the two paths are interchangeable."""

    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        return _gather_blocks(x, group)

    @staticmethod
    def backward(ctx, grad: Tensor):
        return _reduce_scatter_blocks(grad, ctx.group), None


class _ScatterSequence(torch.autograd.Function):
    """Sequence-parallel exit: sum the partial products over the group and keep this rank's token
    block of dim 0 forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x: Tensor, group):
        ctx.group = group
        return _reduce_scatter_blocks(x, group)

    @staticmethod
    def backward(ctx, grad: Tensor):
        return _gather_blocks(grad, ctx.group), None


# --------------------------------------------------------------------------------------------------
# Sharded linears
# --------------------------------------------------------------------------------------------------
class _ParallelLinear(nn.Module):
    def __init__(self, source: nn.Linear, group, rank: int, world: int, shard_dim: int,
                 sequence_parallel: bool) -> None:
        super().__init__()
        full = source.weight.shape[shard_dim]
        if full % world != 0:
            raise ValueError(
                f"cannot shard a dimension of {full} over tensor parallel degree {world}"
            )
        self.group = group
        self.tp_rank = rank
        self.tp_world = world
        self.sequence_parallel = sequence_parallel
        self.in_features = source.in_features
        self.out_features = source.out_features
        self.shard_dim = shard_dim
        shard = source.weight.detach().chunk(world, dim=shard_dim)[rank].clone()
        self.weight = nn.Parameter(shard, requires_grad=source.weight.requires_grad)
        self.weight.tensor_parallel_dim = shard_dim
        self.bias = None
        # Set by ``attach_fused_workspace``: symmetric NVLink buffers shared by the layers of a group.
        self.workspace = None
        # Set by ``attach_peer_runtime``: row-parallel outputs small enough for the one-shot
        # peer-memory all-reduce (decode steps) then skip the c10d collective.
        self.peer_runtime = None

    def _use_fused(self, x: Tensor, rows_local: int) -> bool:
        """Fused collective path: CUDA bf16 fast path, no bias, 128-row aligned token blocks."""
        if self.workspace is None or self.bias is not None or not x.is_cuda:
            return False
        from ohara_b200 import ops
        from ohara_b200.parallel.tp_fused import LazyTPWorkspace, fused_supported

        if not (ops.fast_path(x) and fused_supported(rows_local, *self.weight.shape[::-1])):
            return False
        if isinstance(self.workspace, LazyTPWorkspace):
            self.workspace = self.workspace.materialize(rows_local)
        width = max(self.weight.shape[0] if self.shard_dim == 1 else self.weight.shape[1], 1)
        if rows_local * width > self.workspace.capacity:
            raise ValueError(
                f"a block of {rows_local} x {width} does not fit the tensor-parallel workspace "
                f"({self.workspace.capacity} elements, sized at the first fused call)")
        return True

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"tp={self.tp_world}, local_weight={tuple(self.weight.shape)}")


class ColumnParallelLinear(_ParallelLinear):
    """Output features split over the group; input replicated (or sequence-sharded with SP)."""

    def __init__(self, source: nn.Linear, group, rank: int, world: int,
                 sequence_parallel: bool = False, gather_output: bool = False) -> None:
        super().__init__(source, group, rank, world, 0, sequence_parallel)
        self.gather_output = gather_output
        if source.bias is not None:
            self.bias = nn.Parameter(source.bias.detach().chunk(world)[rank].clone())
            self.bias.tensor_parallel_dim = 0

    def forward(self, x: Tensor) -> Tensor:
        from ohara_b200 import ops

        if self.sequence_parallel and self._use_fused(x, x.numel() // x.shape[-1]):
            from ohara_b200.parallel.tp_fused import column_parallel_fused

            # Token blocks are gathered along dim 0: (B_local, T, in) -> (world * B_local, T, out).
            y = column_parallel_fused(x.reshape(-1, x.shape[-1]), self.weight, self.workspace)
            return y.view(x.shape[0] * self.tp_world, *x.shape[1:-1], self.weight.shape[0])
        if self.sequence_parallel:
            x = _GatherSequence.apply(x, self.group)
        else:
            x = _CopyToGroup.apply(x, self.group)
        y = ops.linear(x, self.weight, self.bias)
        return _GatherFeatures.apply(y, self.group) if self.gather_output else y


class RowParallelLinear(_ParallelLinear):
    """Input features split over the group; partial outputs summed (or reduce-scattered)."""

    def __init__(self, source: nn.Linear, group, rank: int, world: int,
                 sequence_parallel: bool = False) -> None:
        super().__init__(source, group, rank, world, 1, sequence_parallel)
        if source.bias is not None:
            self.bias = nn.Parameter(source.bias.detach().clone())

    def forward(self, x: Tensor) -> Tensor:
        from ohara_b200 import ops

        rows = x.numel() // x.shape[-1]
        if (self.sequence_parallel and rows % self.tp_world == 0 and x.shape[0] % self.tp_world == 0
                and self._use_fused(x, rows // self.tp_world)):
            from ohara_b200.parallel.tp_fused import row_parallel_fused

            # The summed product is scattered in token blocks along dim 0:
            # (B, T, in_local) -> (B / world, T, out).
            y = row_parallel_fused(x.reshape(-1, x.shape[-1]), self.weight, self.workspace)
            return y.view(x.shape[0] // self.tp_world, *x.shape[1:-1], self.weight.shape[0])
        y = ops.linear(x, self.weight, None)
        if self.sequence_parallel:
            y = _ScatterSequence.apply(y, self.group)
        else:
            y = _ReduceFromGroup.apply(y, self.group, self.peer_runtime)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y


def fused_column_parallel(x: Tensor, layers) -> Tensor | None:
    """The outputs of several column-parallel layers that share the input ``x``, concatenated
    along the last dimension and computed by ONE gather + GEMM, when every layer is a bias-free
    :class:`ColumnParallelLinear` on the fused sequence-parallel path; ``None`` otherwise (the
    caller then runs the layers one by one). ``x`` is ``(B_local, T, in)``; the result is
    ``(world * B_local, T, sum of local out_features)``."""
    from ohara_b200 import ops

    first = layers[0]
    if not all(type(layer) is ColumnParallelLinear and layer.bias is None
               and layer.sequence_parallel and layer.workspace is not None
               and layer.group is first.group for layer in layers):
        return None
    if not ops.fused_projections(x):
        return None
    rows_local = x.numel() // x.shape[-1]
    if not first._use_fused(x, rows_local):
        return None
    for layer in layers:  # the first fused call may have materialised the group's workspace
        layer.workspace = first.workspace
    from ohara_b200.parallel.tp_fused import column_parallel_fused_cat

    y = column_parallel_fused_cat(x.reshape(-1, x.shape[-1]),
                                  tuple(layer.weight for layer in layers), first.workspace)
    return y.view(x.shape[0] * first.tp_world, *x.shape[1:-1], y.shape[-1])


def apply_tensor_parallel(module: nn.Module, tp_group=None, plan: TensorParallelPlan | None = None,
                          tp_rank: int | None = None, tp_world: int | None = None, *,
                          tp_mesh=None) -> nn.Module:
    """Replace every ``nn.Linear`` matched by ``plan`` with its sharded counterpart, in place.
    ``tp_mesh`` (the reference's argument: a one-dimensional ``DeviceMesh``,
    ohara/runtime/tensor_parallel.py:65-69) is accepted in place of ``tp_group``; only its
    process group is used, the layers here are not DTensor modules."""
    if tp_mesh is not None:
        if tp_group is not None:
            raise ValueError("pass tp_group or tp_mesh, not both")
        tp_group = tp_mesh.get_group()
    if plan is None:
        raise ValueError("apply_tensor_parallel needs a TensorParallelPlan")
    plan.validate()
    world = tp_world if tp_world is not None else dist.get_world_size(tp_group)
    rank = tp_rank if tp_rank is not None else dist.get_rank(tp_group)
    if plan.degree not in (0, 1, world):
        raise ValueError(f"plan degree {plan.degree} does not match the group size {world}")
    replaced = 0
    for fqn, child in list(module.named_modules()):
        if not fqn or not isinstance(child, nn.Linear):
            continue
        style = plan.style_for(fqn)
        if style is None:
            continue
        parent_name, _, leaf = fqn.rpartition(".")
        parent = module.get_submodule(parent_name) if parent_name else module
        if style == TensorParallelStyle.ROWWISE:
            replacement = RowParallelLinear(child, tp_group, rank, world, plan.sequence_parallel)
        else:
            replacement = ColumnParallelLinear(
                child, tp_group, rank, world, plan.sequence_parallel,
                gather_output=style == TensorParallelStyle.COLWISE_GATHERED)
        setattr(parent, leaf, replacement)
        replaced += 1
    if replaced == 0:
        raise ValueError(
            "No modules matched tensor parallel rules. "
            "Provide matching TensorParallelRule patterns for your model."
        )
    module.tensor_parallel_degree = world
    return module


def attach_fused_workspace(module: nn.Module, workspace) -> int:
    """Give every sharded linear of ``module`` the group's :class:`TPWorkspace`, which switches
    its sequence-parallel collectives to the in-GEMM NVLink path. In that mode activations are
    sharded over dim 0 in whole token blocks (``(B / tp, T, d)`` between the parallel regions).
    Returns the number of layers attached."""
    attached = 0
    for child in module.modules():
        if isinstance(child, _ParallelLinear):
            child.workspace = workspace
            attached += 1
    return attached


def attach_peer_runtime(module: nn.Module, runtime) -> int:
    """Give every row-parallel linear of ``module`` the group's ``PeerRuntime``; returns the number
    of layers attached."""
    attached = 0
    for child in module.modules():
        if isinstance(child, RowParallelLinear):
            child.peer_runtime = runtime
            attached += 1
    return attached


def gather_tensor_parallel_state(module: nn.Module, tp_group) -> dict[str, Tensor]:
    """Full (unsharded) state dict of a tensor-parallel module: shards are all-gathered along the
    dimension recorded on each parameter, so the result loads into a single-device model."""
    world = dist.get_world_size(tp_group)
    sharded = {
        name: getattr(param, "tensor_parallel_dim")
        for name, param in module.named_parameters()
        if hasattr(param, "tensor_parallel_dim")
    }
    full: dict[str, Tensor] = {}
    for name, tensor in module.state_dict().items():
        if name in sharded:
            parts = [torch.empty_like(tensor) for _ in range(world)]
            dist.all_gather(parts, tensor.contiguous(), group=tp_group)
            full[name] = torch.cat(parts, dim=sharded[name])
        else:
            full[name] = tensor
    return full
