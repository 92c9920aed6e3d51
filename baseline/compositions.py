"""Stock-PyTorch compositions around the unmodified reference modules.

The reference engine runs a single device, DDP and a DTensor tensor-parallel plan whose attention
reshape uses the global head count (ohara/models/llama.py:88-90). It has no sharded data
parallelism, no context parallelism and no expert parallelism. For the benchmark configurations
that name those, the reference-equivalent arm is the reference's own modules, optimizers and
trainer composed with what stock PyTorch offers:

``TensorParallelFSDPEngine``
    the reference engine and its tensor-parallel plan (ohara/runtime/tensor_parallel.py:34-48,
    ``parallelize_module`` with ``ColwiseParallel`` / ``RowwiseParallel``), the attention modules'
    head counts divided by the degree (the one-line correction of the reshape), and
    ``torch.distributed.fsdp.fully_shard`` per block + root over the data-parallel mesh dimension.
``ContextParallelEngine``
    ``fully_shard`` over all ranks and every forward / backward inside
    ``torch.distributed.tensor.experimental.context_parallel`` (ring SDPA with load balancing),
    which shards the token, target and rotary buffers along the sequence.
``ExpertParallelEngine``
    the reference ``GroupedMoE`` keeps ``E / world`` experts per rank; its grouped dispatch is
    replaced by: sort pairs by expert, exchange counts and rows with ``all_to_all_single``, run the
    same three ``torch._grouped_mm`` calls on the received rows, send the results back and combine.
    Dense parameters go through the reference's DDP strategy, expert parameters are left out of it.

Nothing here imports this repository's package.
"""

from __future__ import annotations

import contextlib
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F


def describe(spec: dict, world: int) -> str:
    if world == 1:
        return "single"
    parts = []
    if spec["tp"] > 1:
        parts.append(f"tp{spec['tp']} (DTensor)")
    if spec["cp"] > 1:
        parts.append(f"cp{spec['cp']} (ring SDPA)")
    if spec["ep"] > 1:
        parts.append(f"ep{spec['ep']} (all_to_all_single)")
    if spec["tp"] > 1 or spec["cp"] > 1:
        parts.append(f"fully_shard{spec['dp'] * spec['cp']}")
    else:
        parts.append(f"ddp{world}")
    return " x ".join(parts)


def data_rank(engine) -> tuple[int, int]:
    """(rank, world) that decide which data a process sees."""
    override = getattr(engine, "data_rank_world", None)
    if override is not None:
        return override
    topo = engine.topology
    if getattr(engine, "_dp_world_size", 1) > 1:
        return engine._dp_rank, engine._dp_world_size
    return 0, 1


def build_engine(spec: dict):
    from ohara import OharaEngine
    from ohara.runtime import EngineConfig, ParallelConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 or (spec["tp"] == 1 and spec["cp"] == 1 and spec["ep"] == 1):
        return OharaEngine(), "reference as shipped"
    if spec["tp"] > 1:
        config = EngineConfig(parallel=ParallelConfig(tp=spec["tp"]))
        return (TensorParallelFSDPEngine(config),
                "reference-equivalent: reference tensor-parallel plan + head-count correction + "
                "fully_shard")
    if spec["cp"] > 1:
        return (ContextParallelEngine(EngineConfig(), spec),
                "reference-equivalent: context_parallel ring SDPA + fully_shard")
    return (ExpertParallelEngine(EngineConfig()),
            "reference-equivalent: reference GroupedMoE sharded over ranks, all_to_all_single "
            "dispatch / combine, DDP for dense parameters")


def _reference_engine_class():
    from ohara import OharaEngine

    return OharaEngine


def _bf16_policy():
    from torch.distributed.fsdp import MixedPrecisionPolicy

    return MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)


class _NoSyncMixin:
    """Gradient accumulation for ``fully_shard`` modules: skip the reduce-scatter except on the
    last micro-batch (the counterpart of DDP's ``no_sync``)."""

    def no_backward_sync(self, module, enabled: bool = True):
        @contextlib.contextmanager
        def scope():
            setter = getattr(module, "set_requires_gradient_sync", None)
            if callable(setter) and enabled:
                setter(False)
                try:
                    yield
                finally:
                    setter(True)
            else:
                yield

        return scope()

    def no_sync(self, module, enabled: bool = True):
        return self.no_backward_sync(module, enabled)

    def autocast_context(self):
        # fully_shard's mixed-precision policy casts parameters; activations follow autocast as
        # in the reference's bf16_mixed mode
        if self.device.type == "cuda":
            return torch.autocast("cuda", dtype=torch.bfloat16)
        return contextlib.nullcontext()


def _shard_blocks(model, mesh):
    from torch.distributed.fsdp import fully_shard

    policy = _bf16_policy()
    for block in model.layers:
        fully_shard(block, mesh=mesh, mp_policy=policy)
    fully_shard(model, mesh=mesh, mp_policy=policy)
    return model


class TensorParallelFSDPEngine(_NoSyncMixin, _reference_engine_class()):
    def prepare_module(self, module, *, move_to_device: bool = True):
        from ohara.runtime.tensor_parallel import TensorParallelPlan, apply_tensor_parallel
        from torch.distributed.device_mesh import init_device_mesh

        self.launch()
        if move_to_device:
            module = module.to(self._device)
        # every rank must shard the same initial weights
        for tensor in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(tensor.data, src=0)
        tp = self.topology.tp
        dp = dist.get_world_size() // tp
        # same rank order as the reference topology: tensor-parallel peers are neighbours
        mesh = init_device_mesh(self._device.type, (dp, tp), mesh_dim_names=("dp", "tp"))
        # the reference's own plan and its own parallelize_module call
        module = apply_tensor_parallel(module, mesh["tp"], TensorParallelPlan.llama_default(tp))
        for block in module.layers:
            attn = block.attn
            # the reshape at ohara/models/llama.py:88-90 needs the *local* head counts
            attn.num_attention_heads //= tp
            attn.num_key_value_heads //= tp
        if dp > 1:
            module = _shard_blocks(module, mesh["dp"])
        self.data_rank_world = (dist.get_rank() // tp, dp)
        return module


class _SequenceShardedModel(torch.nn.Module):
    """Runs the wrapped reference model on this rank's shard of every sequence: inside
    ``context_parallel`` the token ids and the rotary tables are cut along the sequence (with the
    load-balancing permutation) and ``scaled_dot_product_attention`` becomes ring attention. The
    backward of ring attention is part of the autograd graph, so leaving the region after the
    forward is fine."""

    def __init__(self, inner, mesh, seq_len: int) -> None:
        super().__init__()
        self.inner, self.mesh, self.seq_len = inner, mesh, seq_len
        self.config = inner.config
        self._cos = inner.freq_cos[:seq_len].clone()
        self._sin = inner.freq_sin[:seq_len].clone()

    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.inner.set_requires_gradient_sync(flag)

    def forward(self, data):
        from torch.distributed.tensor.experimental import context_parallel

        data = data.clone()
        # the model slices its rotary tables by local length from row 0: hand it tables that hold
        # exactly the rows of this rank's positions
        cos, sin = self._cos.clone(), self._sin.clone()
        with context_parallel(self.mesh, buffers=[data, cos, sin], buffer_seq_dims=[1, 0, 0],
                              no_restore_buffers={data, cos, sin}):
            self.inner.freq_cos, self.inner.freq_sin = cos, sin
            return self.inner(data)


class ContextParallelEngine(_NoSyncMixin, _reference_engine_class()):
    def __init__(self, config, spec: dict) -> None:
        super().__init__(config)
        self._spec = spec

    def prepare_module(self, module, *, move_to_device: bool = True):
        from torch.distributed.device_mesh import init_device_mesh

        self.launch()
        if move_to_device:
            module = module.to(self._device)
        for tensor in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(tensor.data, src=0)
        world = dist.get_world_size()
        self._cp_mesh = init_device_mesh(self._device.type, (world,), mesh_dim_names=("cp",))
        module = _shard_blocks(module, self._cp_mesh)
        self.data_rank_world = (0, 1)  # every rank of the group works on the same sequences
        self._dp_world_size, self._dp_rank = 1, 0
        return _SequenceShardedModel(module, self._cp_mesh, self._spec["seq_len"])

    def to_device(self, value):
        """Batches are ``(tokens, targets)``: tokens go to the device whole (the model wrapper
        shards them), targets are cut to this rank's positions with the same permutation."""
        from torch.distributed.tensor.experimental import context_parallel

        if isinstance(value, (tuple, list)) and len(value) == 2:
            data = value[0].to(self._device, non_blocking=True)
            target = value[1].to(self._device, non_blocking=True)
            if target.shape[1] == self._spec["seq_len"]:  # not cut yet (loaders call this too)
                target = target.clone()
                with context_parallel(self._cp_mesh, buffers=[target], buffer_seq_dims=[1],
                                      no_restore_buffers={target}):
                    pass
            return type(value)((data, target))
        return super().to_device(value)


class ExpertParallelEngine(_reference_engine_class()):
    def prepare_module(self, module, *, move_to_device: bool = True):
        from ohara.modules.moe_grouped import GroupedMoE
        from torch.nn.parallel import DistributedDataParallel

        self.launch()
        if move_to_device:
            module = module.to(self._device)
        for tensor in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(tensor.data, src=0)
        world, rank = dist.get_world_size(), dist.get_rank()
        ignored = []
        for name, layer in module.named_modules():
            if isinstance(layer, GroupedMoE):
                shard_experts(layer, rank, world)
                ignored += [f"{name}.{p}" for p in ("w_gate", "w_up", "w_down")]
        DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(module, ignored)
        return self._strategy.setup_module(module, device=self._device, process_group=None)


# --------------------------------------------------------------------------------------------------
# Expert parallelism around the reference GroupedMoE
# --------------------------------------------------------------------------------------------------
def shard_experts(layer, rank: int, world: int) -> None:
    """Keep ``E / world`` experts of ``layer`` and replace its grouped dispatch by the
    all-to-all version. Expert gradients sum the contributions of every rank's tokens, so they
    are scaled by ``1 / world`` to match the rank-averaged loss that DDP optimises."""
    local = layer.num_experts // world
    for name in ("w_gate", "w_up", "w_down"):
        full = getattr(layer, name)
        shard = torch.nn.Parameter(full.detach()[rank * local:(rank + 1) * local].clone())
        shard.register_hook(lambda grad, s=1.0 / world: grad * s)
        setattr(layer, name, shard)
    layer._ep_world, layer._ep_local = world, local
    layer._dispatch_grouped = _dispatch_all_to_all.__get__(layer)
    layer._dispatch_reference = layer._dispatch_grouped  # CPU: same exchange, per-expert loop


def _all_to_all(x: torch.Tensor, out_splits: list[int], in_splits: list[int]) -> torch.Tensor:
    from torch.distributed._functional_collectives import all_to_all_single_autograd

    return all_to_all_single_autograd(x, out_splits, in_splits, dist.group.WORLD)


def _dispatch_all_to_all(self, flat_x, expert_indices, expert_weights):
    """ohara/modules/moe_grouped.py:156-185 with the expert dimension sharded over the ranks."""
    world, local = self._ep_world, self._ep_local
    k = self.num_experts_per_tok
    flat_indices = expert_indices.reshape(-1)
    order = torch.argsort(flat_indices, stable=True)      # pairs sorted by (global) expert
    rows = order // k
    counts = torch.bincount(flat_indices, minlength=self.num_experts)
    # counts table: what every rank sends to each of my experts
    received = torch.empty_like(counts)
    dist.all_to_all_single(received, counts)               # (world, local) flattened, by source
    send_splits = counts.view(world, local).sum(1).tolist()
    received = received.view(world, local)
    recv_splits = received.sum(1).tolist()
    compute_dtype = (torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda")
                     else flat_x.dtype)
    x_sorted = flat_x[rows].to(compute_dtype)
    x_recv = _all_to_all(x_sorted, recv_splits, send_splits)
    # received rows are ordered (source, expert); the grouped product wants them by expert
    expert_of_row = torch.repeat_interleave(
        torch.arange(local, device=flat_x.device).repeat(world), received.reshape(-1))
    by_expert = torch.argsort(expert_of_row, stable=True)
    offsets = received.sum(0).cumsum(0).to(torch.int32)
    x_local = x_recv[by_expert]
    if x_local.is_cuda:
        gate = torch._grouped_mm(x_local, self.w_gate.to(compute_dtype), offs=offsets)
        up = torch._grouped_mm(x_local, self.w_up.to(compute_dtype), offs=offsets)
        hidden = F.silu(gate) * up
        y_local = torch._grouped_mm(hidden, self.w_down.to(compute_dtype), offs=offsets)
    else:  # no grouped kernel on CPU: the same products expert by expert
        pieces, begin = [], 0
        for expert, end in enumerate(offsets.tolist()):
            xe = x_local[begin:end]
            he = F.silu(xe @ self.w_gate[expert].to(xe.dtype)) * (xe @ self.w_up[expert].to(xe.dtype))
            pieces.append(he @ self.w_down[expert].to(xe.dtype))
            begin = end
        y_local = torch.cat(pieces) if pieces else x_local.new_zeros(0, flat_x.shape[1])
    y_recv = torch.empty_like(y_local)
    y_recv[by_expert] = y_local
    y = _all_to_all(y_recv, send_splits, recv_splits)
    y = y * expert_weights.reshape(-1)[order].unsqueeze(-1).to(y.dtype)
    out = torch.zeros_like(flat_x)
    out.index_add_(0, rows, y.to(out.dtype))
    return out


def apply_router_skew(model, spec: dict, cfg, device) -> None:
    """The same forced selection bias as the other arm: half of every token's picks go to a few
    experts of the first rank."""
    from ohara.modules.moe_grouped import GroupedMoE

    from bench import force_router_skew

    force_router_skew(model, GroupedMoE, spec["model"]["moe_experts_per_tok"])
