"""``OharaEngine``: the runtime facade the trainer talks to.

Same surface as the reference engine (ohara/runtime/engine.py:57-499) — ``launch``, ``prepare`` /
``setup`` aliases, ``prepare_dataloaders``, ``to_device``, ``autocast_context``, ``backward``,
``no_backward_sync``, ``clip_gradients``, ``optimizer_step``, collectives, atomic ``save`` /
``load``, ``log_dict`` — with a different engine room:

* one process per GPU; c10d (NCCL, or gloo without CUDA) is the control plane;
* process groups exist for every parallel dimension (data, tensor, context, expert), built from
  :class:`ParallelTopology` arithmetic rather than a DeviceMesh;
* tensor parallelism replaces the matched linears by sharded modules (no DTensor);
* data parallelism is DDP or the sharded-optimizer strategy (``StrategyType.FSDP``), whose
  reduce-scatter / optimizer / all-gather run as fused peer-memory kernels when enabled;
* batches move host→device through pinned staging on a side stream.
"""

from __future__ import annotations

import os
from collections.abc import Callable, Mapping
from contextlib import nullcontext
from datetime import timedelta
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist
from torch.optim import Optimizer
from torch.utils.data import DataLoader, DistributedSampler, IterableDataset, RandomSampler

from .config import EngineConfig
from .enums import Backend, PrecisionMode, ReduceType, StrategyType
from .strategy import BaseStrategy, DDPStrategy, FSDPStrategy, SingleStrategy
from .tensor_parallel import (
    attach_fused_workspace,
    attach_peer_runtime,
    TensorParallelPlan,
    apply_tensor_parallel,
    gather_tensor_parallel_state,
)
from .topology import ParallelTopology
from .watchdog import Heartbeat, StepWatchdog, default_store


class _DeviceDataLoader:
    """Iterates a dataloader and yields batches already on the engine's device."""

    def __init__(self, dataloader: DataLoader, engine: "OharaEngine") -> None:
        self.dataloader = dataloader
        self.engine = engine
        self.epoch = 0

    def __iter__(self):
        sampler = getattr(self.dataloader, "sampler", None)
        if isinstance(sampler, DistributedSampler):
            sampler.set_epoch(self.epoch)
            self.epoch += 1
        for batch in self.dataloader:
            yield self.engine.to_device(self.engine.local_batch(batch))

    def __len__(self) -> int:
        return len(self.dataloader)

    def __getattr__(self, name: str) -> Any:
        return getattr(self.dataloader, name)


_REDUCE_OPS = {
    ReduceType.SUM: "SUM",
    ReduceType.MEAN: "SUM",
    ReduceType.MAX: "MAX",
    ReduceType.MIN: "MIN",
}


def _strip_wrapper_prefixes(name: str) -> str:
    changed = True
    while changed:
        changed = False
        for prefix in ("module.", "_orig_mod."):
            if name.startswith(prefix):
                name, changed = name[len(prefix):], True
    return name


def _stage_to_model_name(name: str, first_layer: int) -> str:
    """``layers.<i>.…`` of a pipeline stage is ``layers.<first_layer + i>.…`` of the model."""
    if name.startswith("layers."):
        index, rest = name.split(".", 2)[1:]
        return f"layers.{int(index) + first_layer}.{rest}"
    return name


class OharaEngine:
    def __init__(self, config: EngineConfig | None = None, loggers: list[Any] | None = None) -> None:
        self.config = config or EngineConfig()
        self.loggers = loggers or []
        self._launched = False
        self._device = torch.device("cpu")
        self._strategy: BaseStrategy = SingleStrategy()
        try:
            self.topology = ParallelTopology.from_config(1, self.config.parallel)
        except ValueError:
            self.topology = ParallelTopology(1, 1, 1, 1, 1, 1, 1)
        self._scaler = self._build_grad_scaler(False)
        self._groups: dict[str, Any] = {}
        self._dp_world_size = 1
        self._dp_rank = 0
        self.heartbeat: Heartbeat | None = None
        self.watchdog: StepWatchdog | None = None

    # -- properties ----------------------------------------------------------------------------
    @staticmethod
    def _build_grad_scaler(enabled: bool):
        return torch.amp.GradScaler("cuda", enabled=enabled)

    @property
    def launched(self) -> bool:
        return self._launched

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def world_size(self) -> int:
        return self.topology.world_size

    @property
    def global_rank(self) -> int:
        return self.topology.global_rank

    @property
    def is_global_zero(self) -> bool:
        return self.global_rank == 0

    @property
    def data_parallel_rank(self) -> int:
        """Rank used to shard input data; tensor/context-parallel peers share it, expert-parallel
        peers do not (they route their own tokens)."""
        return self.topology.dp_rank * self.topology.ep + self.topology.ep_rank

    @property
    def data_parallel_world_size(self) -> int:
        return self.topology.dp_world_size * self.topology.ep

    @property
    def strategy(self) -> BaseStrategy:
        return self._strategy

    def group(self, name: str):
        """Process group of a parallel dimension: ``"dp"``, ``"tp"``, ``"cp"`` or ``"ep"``
        (``None`` = the default world group, or no group when not distributed)."""
        return self._groups.get(name)

    # -- launch --------------------------------------------------------------------------------
    def launch(self, function: Callable[..., Any] | None = None, *args: Any, **kwargs: Any) -> Any:
        if not self._launched:
            self._do_launch()
        if function is not None:
            return function(*args, **kwargs)
        return None

    def _do_launch(self) -> None:
        world_size = int(os.environ.get("WORLD_SIZE", "1"))
        wants_dist = world_size > 1 or int(os.environ.get("RANK", "0")) > 0
        backend_name: str | None = None
        if wants_dist and not dist.is_initialized():
            backend = self.config.distributed.backend
            if backend == Backend.NCCL and not torch.cuda.is_available():
                backend = Backend.GLOO
            if torch.cuda.is_available() and backend == Backend.NCCL:
                local_rank = int(os.environ.get("LOCAL_RANK", "0"))
                if local_rank < torch.cuda.device_count():
                    torch.cuda.set_device(local_rank)
            dist.init_process_group(
                backend=backend.value,
                timeout=timedelta(seconds=self.config.distributed.timeout_seconds),
            )
        if dist.is_initialized():
            world_size = dist.get_world_size()
            backend_name = dist.get_backend()
        self.topology = ParallelTopology.from_config(world_size, self.config.parallel)

        if torch.cuda.is_available() and (not wants_dist or backend_name == Backend.NCCL.value):
            self._device = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
            torch.cuda.set_device(self._device)
        elif torch.backends.mps.is_available():
            self._device = torch.device("mps")
        else:
            self._device = torch.device("cpu")

        strategy = self.config.strategy
        if strategy == StrategyType.AUTO:
            replicas = self.topology.dp_enabled or self.topology.ep > 1
            strategy = StrategyType.DDP if replicas else StrategyType.SINGLE
        if strategy in (StrategyType.DDP, StrategyType.FSDP) and not self.topology.distributed_enabled:
            strategy = StrategyType.SINGLE if strategy == StrategyType.DDP else strategy
        self._build_groups()
        data_parallel = strategy in (StrategyType.DDP, StrategyType.FSDP)
        # expert-parallel peers route their own tokens: for data they count as replicas
        self._dp_world_size = self.topology.dp_world_size * self.topology.ep if data_parallel else 1
        self._dp_rank = (self.topology.dp_rank * self.topology.ep + self.topology.ep_rank
                         if data_parallel else 0)
        if self.config.shard_parameters and strategy != StrategyType.FSDP:
            raise ValueError("shard_parameters needs the sharded strategy (StrategyType.FSDP); "
                             f"this engine resolved to {strategy.value!r}")
        if strategy == StrategyType.DDP:
            self._strategy = DDPStrategy(init_sync=not self.topology.tp_enabled)
        elif strategy == StrategyType.FSDP:
            fused = self.config.fused_collectives and self._device.type == "cuda"
            topo = self.topology
            # With tensor / expert parallelism the shards differ between ranks of the optimizer's
            # group: the engine then equalises the full model before it is sharded instead.
            composed = topo.tp_enabled or topo.ep > 1 or topo.cp > 1 or topo.pp > 1
            hybrid = topo.dp_replicate > 1 and topo.dp_shard > 1
            if self.config.shard_parameters and (topo.ep > 1 or topo.pp > 1):
                raise NotImplementedError("shard_parameters composes with data (plain or hybrid), "
                                          "tensor and context parallelism, not with ep / pp")
            self._strategy = FSDPStrategy(fused=fused, init_sync=not composed,
                                          shard_parameters=self.config.shard_parameters,
                                          shard_parameters_layout=self.config.shard_parameters_layout)
            base_size = topo.dp_shard if hybrid else topo.dp_world_size
            norm_groups = {}
            if topo.tp_enabled:
                norm_groups["tp"] = self._groups.get("tp")
            if topo.ep > 1:
                norm_groups["ep"] = self._groups.get("ep")
            if topo.pp > 1:
                norm_groups["pp"] = self._groups.get("pp")
            self._strategy.configure(
                replicate_group=self._groups.get("replicate"),
                replicate_world=topo.dp_replicate if hybrid else 1,
                expert_parallel=topo.ep > 1,
                expert_group=self._groups.get("expert_shard"),
                expert_world=base_size * topo.cp,
                norm_groups=norm_groups,
                shard_world=base_size * topo.cp * topo.ep,
            )
            self._sharded_over_cp = topo.cp > 1
        else:
            self._strategy = SingleStrategy()
        use_scaler = (
            self.config.precision.mode == PrecisionMode.FP16_MIXED and self._device.type == "cuda"
        )
        self._scaler = self._build_grad_scaler(use_scaler)
        self._start_failure_detection()
        self._launched = True

    def _start_failure_detection(self) -> None:
        tolerance = self.config.fault_tolerance
        store = default_store()
        if tolerance.heartbeat_interval_s > 0 and store is not None and self.world_size > 1:
            self.heartbeat = Heartbeat(
                store, self.global_rank, self.world_size,
                interval_s=tolerance.heartbeat_interval_s, timeout_s=tolerance.heartbeat_timeout_s,
            ).start()
        if tolerance.step_timeout_s > 0:
            # On expiry the copy streams' stream-ordered waits are released first, so that a
            # process that is not ended here can still drain its streams.
            self.watchdog = StepWatchdog(tolerance.step_timeout_s,
                                         on_timeout=lambda step, elapsed: self.abort_fused_waits(),
                                         hard_exit=tolerance.exit_on_step_timeout)

    def check_peers(self, *, refresh: bool = False) -> None:
        """Raise ``PeerFailure`` if a rank of the job is known to be gone. The trainer calls this
        on the host before it launches a step, so that no kernel or collective is issued that
        would wait for the missing rank."""
        if self.heartbeat is not None:
            try:
                self.heartbeat.check(refresh=refresh)
            except Exception:
                self.abort_fused_waits()
                raise

    def guard_step(self, index: int):
        """Context manager that arms the step watchdog (a no-op when none is configured)."""
        if self.watchdog is None:
            return nullcontext()
        return self.watchdog.step(index)

    def check_device_status(self) -> None:
        """Raise ``CollectiveTimeout`` if a kernel of this process gave up a bounded wait (a peer
        flag that never came, a pipeline hand-off that timed out) since the last check. Reads the
        device status word, so call it after a ``synchronize()``: the trainer does so at the end
        of every step and before it writes a checkpoint, which keeps a step whose
        reduce-scatter or all-gather was abandoned from being trained on or saved. On a timeout
        the stream-ordered waits of the fused tensor / context-parallel paths are released first,
        so that the process can still drain its streams and exit. A no-op without CUDA."""
        if self._device.type != "cuda":
            return
        from ohara_b200 import ops
        from ohara_b200.errors import CollectiveTimeout

        try:
            ops.check_status()
        except CollectiveTimeout:
            self.abort_fused_waits()
            raise

    def abort_fused_waits(self) -> int:
        """Release every stream-ordered wait that the fused tensor-parallel and context-parallel
        workspaces of the prepared module may have queued (see ``TPWorkspace.abort``). Called on
        the timeout, peer-failure and watchdog paths; returns the number of workspaces released."""
        module = getattr(self, "_module", None)
        if module is None:
            return 0
        seen: set[int] = set()
        for child in module.modules():
            for name in ("workspace", "cp_workspace"):
                workspace = getattr(child, name, None)
                workspace = getattr(workspace, "workspace", workspace)  # lazy wrappers
                abort = getattr(workspace, "abort", None)
                if callable(abort) and id(workspace) not in seen:
                    seen.add(id(workspace))
                    abort()
        return len(seen)

    def leave(self) -> None:
        """Announce that this rank stops on purpose (between steps, nothing in flight)."""
        if self.heartbeat is not None:
            self.heartbeat.leave()

    def _build_groups(self) -> None:
        """Create one process group per parallel dimension that is larger than 1. Every rank calls
        ``new_group`` for every group of a dimension (a c10d requirement)."""
        self._groups = {}
        topo = self.topology
        if not dist.is_initialized() or topo.world_size <= 1:
            return
        dims = {
            "dp": (("dp_replicate", "dp_shard"), topo.dp_world_size),
            "dp_ep": (("dp_replicate", "dp_shard", "ep"), topo.dp_world_size * topo.ep),
            "tp": (("tp",), topo.tp),
            "cp": (("cp",), topo.cp),
            "ep": (("ep",), topo.ep),
            "pp": (("pp",), topo.pp),
        }
        if self._wants_sharded_optimizer():
            # Groups of the sharded optimizer. Context-parallel and expert-parallel peers hold
            # replicas of the dense parameters, so those are sharded over them as well; the
            # routed experts only over the ranks that hold the same experts. With hybrid sharding
            # (both data-parallel dimensions > 1) ``dp_replicate`` is a replica dimension of its
            # own, otherwise it is folded into the shard group.
            hybrid = topo.dp_replicate > 1 and topo.dp_shard > 1
            base = ("dp_shard",) if hybrid else ("dp_replicate", "dp_shard")
            base_size = topo.dp_shard if hybrid else topo.dp_world_size
            dims["shard"] = ((*base, "cp", "ep"), base_size * topo.cp * topo.ep)
            dims["expert_shard"] = ((*base, "cp"), base_size * topo.cp)
            if hybrid:
                dims["replicate"] = (("dp_replicate",), topo.dp_replicate)
        me = topo.global_rank
        for name, (axes, size) in dims.items():
            if size <= 1:
                continue
            if size == topo.world_size:
                self._groups[name] = None  # the default group
                continue
            for ranks in topo.iter_groups(axes):
                pg = dist.new_group(ranks=ranks)
                if me in ranks:
                    self._groups[name] = pg

    def _wants_sharded_optimizer(self) -> bool:
        return self.config.strategy == StrategyType.FSDP

    # -- prepare -------------------------------------------------------------------------------
    def prepare(self, module: torch.nn.Module, *optimizers: Optimizer):
        module = self.prepare_module(module)
        if not optimizers:
            return module
        wrapped = self.prepare_optimizers(*optimizers)
        if len(wrapped) == 1:
            return module, wrapped[0]
        return (module, *wrapped)

    def prepare_module(self, module: torch.nn.Module, *, move_to_device: bool = True) -> torch.nn.Module:
        self.launch()
        if move_to_device:
            if self.config.precision.mode == PrecisionMode.BF16_TRUE:
                module = module.to(device=self._device, dtype=torch.bfloat16)
            else:
                module = module.to(self._device)
        self._equalise_initial_weights(module)
        if self.config.activation_checkpointing:
            enable = getattr(module, "enable_activation_checkpointing", None)
            if not callable(enable):
                raise ValueError("activation_checkpointing needs a model that offers "
                                 "enable_activation_checkpointing() (Llama)")
            enable(True)
        module = self._maybe_apply_tensor_parallel(module)
        module = self._maybe_apply_pipeline_parallel(module)
        self._maybe_apply_context_parallel(module)
        ignored = self._maybe_apply_expert_parallel(module)
        if ignored and isinstance(self._strategy, DDPStrategy):
            from torch.nn.parallel import DistributedDataParallel

            DistributedDataParallel._set_params_and_buffers_to_ignore_for_model(module, ignored)
        if isinstance(self._strategy, FSDPStrategy):
            group = self._groups.get("shard")
        else:
            group = self._groups.get("dp_ep") if self.topology.ep > 1 else self._groups.get("dp")
        replicas = self.topology.dp_world_size * (self.topology.ep if self.topology.ep > 1 else 1)
        if isinstance(self._strategy, DDPStrategy) and replicas <= 1:
            # every other rank of the job is a tensor- / context- / pipeline-parallel peer: there
            # is nothing to replicate over, and the default group would average different shards
            self._module = module
            return module
        module = self._strategy.setup_module(module, device=self._device, process_group=group)
        sharding = getattr(module, "_param_sharding", None)
        if sharding is not None and getattr(self, "_tp_batch_sharding", False):
            # sequence-parallel layout: replicated parameters hold partial gradients per tp rank
            sharding.partial_gradient_group = self._groups.get("tp")
            sharding.partial_gradients = True
        self._module = module
        return module

    def _maybe_apply_pipeline_parallel(self, module: torch.nn.Module) -> torch.nn.Module:
        """With ``pp > 1`` this rank keeps one contiguous run of the model's blocks (the embedding
        on the first stage, the final norm and the output projection on the last) and the module
        handed back drives the pipeline: its forward runs every micro-batch of the batch through
        this stage and returns the loss of the step, ``backward`` on that loss runs the backward
        passes (see :class:`ohara_b200.parallel.pipeline.PipelinedLlama`). Micro-batches are
        ``config.pipeline.micro_batch_size`` sequences."""
        if self.topology.pp <= 1:
            return module
        from ohara_b200.parallel.pipeline import LlamaStage, PipelinedLlama

        if not all(hasattr(module, name) for name in ("layers", "token_emb", "vocab_proj", "norm")):
            raise ValueError("pp > 1 needs a Llama-style model (token_emb, layers, norm, vocab_proj)")
        if self.topology.cp > 1 or self.topology.ep > 1:
            raise NotImplementedError("pipeline parallelism composes with data and tensor "
                                      "parallelism only")
        flops = float(module.estimate_flops()) if hasattr(module, "estimate_flops") else 0.0
        stage = LlamaStage(module, self.topology.pp, self.topology.pp_rank)
        wrapped = PipelinedLlama(stage, self._groups.get("pp"),
                                 self.config.pipeline.micro_batch_size)
        wrapped._model_flops = flops
        return wrapped

    def _equalise_initial_weights(self, module: torch.nn.Module) -> None:
        """With the sharded optimizer composed with tensor / expert / context parallelism every
        rank first holds the whole model: broadcast rank 0's values so that all shards are cut
        from the same weights (the per-group broadcast that plain data parallelism uses would
        overwrite one rank's expert or tensor shard with another's)."""
        composed_fsdp = isinstance(self._strategy, FSDPStrategy) and not self._strategy.init_sync
        if not (composed_fsdp or self.topology.pp > 1):
            return
        if not dist.is_initialized() or self.topology.world_size <= 1:
            return
        for tensor in list(module.parameters()) + list(module.buffers()):
            dist.broadcast(tensor.data, src=0)

    def _maybe_apply_context_parallel(self, module: torch.nn.Module) -> None:
        """With ``cp > 1`` the ranks of a context-parallel group share a batch and each works on
        one contiguous chunk of every sequence; attention exchanges keys / values over NVLink."""
        if self.topology.cp <= 1:
            return
        enable = getattr(module, "enable_context_parallel", None)
        if not callable(enable):
            raise RuntimeError("cp > 1 needs a model with enable_context_parallel")
        mode = self.config.context_parallel_mode
        if mode == "ulysses":
            # all-to-all over heads: the process group's collective, so CPU ranks work as well
            from ohara_b200.parallel.ulysses import UlyssesWorkspace

            workspace = UlyssesWorkspace(self._groups.get("cp"))
        elif mode == "ring":
            if self._device.type != "cuda":
                raise RuntimeError("the key/value-exchange mode of context parallelism needs CUDA "
                                   "devices (context_parallel_mode='ulysses' runs anywhere)")
            from ohara_b200.parallel.cp import LazyCPWorkspace

            workspace = LazyCPWorkspace(self._groups.get("cp"))
        else:
            raise ValueError(f"unknown context_parallel_mode {mode!r} (ring or ulysses)")
        enable(workspace, self.topology.cp_rank, self.topology.cp)
        self._cp_sequence_sharding = True
        self._replica_grads_synced = True

    def _maybe_apply_expert_parallel(self, module: torch.nn.Module) -> list[str]:
        """With ``ep > 1`` every grouped mixture-of-experts layer keeps ``E / ep`` experts and
        exchanges tokens over NVLink peer memory; expert-parallel peers see different data, so for
        all other parameters they are ordinary data-parallel replicas. Returns the names of the
        expert parameters, which the data-parallel wrapper must leave alone (their gradients are
        averaged over the ``dp`` group separately)."""
        if self.topology.ep <= 1:
            return []
        from ohara_b200.modules.moe_grouped import GroupedMoE
        from ohara_b200.parallel.ep import LazyEPWorkspace

        layers = [m for m in module.modules() if isinstance(m, GroupedMoE)]
        if not layers:
            raise ValueError("ep > 1 but the model has no grouped mixture-of-experts layer")
        peer_memory = self._device.type == "cuda" and self.config.fused_collectives
        shared: dict[tuple[int, int], Any] = {}
        for index, layer in enumerate(layers):
            key = (layer.num_experts, layer.dim)
            if key not in shared and peer_memory:
                shared[key] = LazyEPWorkspace(self._groups.get("ep"), layer.num_experts, layer.dim,
                                              self.config.expert_capacity_factor)
            elif key not in shared:
                # no peer memory (CPU ranks, or fused collectives switched off): the same layer
                # over the group's all-to-all
                from ohara_b200.parallel.ep_c10d import C10dEPWorkspace

                shared[key] = C10dEPWorkspace(self._groups.get("ep"), layer.num_experts)
            layer.shard_experts(shared[key], slot=index)
            topo = self.topology
            sharded = isinstance(self._strategy, FSDPStrategy)
            if layer.quantile_balancing and (sharded or topo.cp == 1):
                # balance on the quantile over the tokens of every rank that routes through
                # these experts (or replicas of them), not on an average of per-rank quantiles
                layer.qb_global = True
                layer.qb_global_group = self._groups.get("shard" if sharded else "dp_ep")
                layer.qb_global_world = topo.dp_world_size * topo.ep * (topo.cp if sharded else 1)
        self._expert_parallel = True
        return [name for name, p in module.named_parameters() if getattr(p, "expert_parallel", False)]

    def sync_expert_gradients(self, model: torch.nn.Module) -> None:
        """Average expert gradients over the data-parallel replicas of each expert shard."""
        if not getattr(self, "_expert_parallel", False) or self.topology.dp_world_size <= 1:
            return
        if isinstance(self._strategy, FSDPStrategy):
            return  # the expert part of the sharded optimizer averages them itself
        group, size = self._groups.get("dp"), self.topology.dp_world_size
        for param in model.parameters():
            if getattr(param, "expert_parallel", False) and param.grad is not None:
                dist.all_reduce(param.grad, group=group)
                param.grad.div_(size)

    def prepare_optimizers(self, *optimizers: Optimizer):
        self.launch()
        module = getattr(self, "_module", None)
        if self.topology.tp_enabled:
            # whole-matrix algorithms (Muon) gather the shards of a matrix over this group
            for opt in optimizers:
                opt.tensor_parallel_group = self._groups.get("tp")
                opt.tensor_parallel_world = self.topology.tp
        wrapped = tuple(self._strategy.setup_optimizer(opt, module) for opt in optimizers)
        for opt in wrapped:
            if callable(getattr(opt, "sync_master_weights", None)):
                self._sharded_optimizer = opt
        return wrapped

    # Fabric-style aliases
    def setup(self, module: torch.nn.Module, *optimizers: Optimizer):
        return self.prepare(module, *optimizers)

    def setup_module(self, module: torch.nn.Module, *, move_to_device: bool = True):
        return self.prepare_module(module, move_to_device=move_to_device)

    def setup_optimizers(self, *optimizers: Optimizer):
        return self.prepare_optimizers(*optimizers)

    def setup_dataloaders(self, *dataloaders: DataLoader):
        return self.prepare_dataloaders(*dataloaders)

    def _resolve_tensor_parallel_plan(self, module: torch.nn.Module) -> TensorParallelPlan:
        plan = self.config.tensor_parallel
        if not self.topology.tp_enabled:
            return plan
        if plan.degree in (0, 1):
            plan = TensorParallelPlan.llama_default(self.topology.tp, plan.sequence_parallel)
        if plan.degree != self.topology.tp:
            raise ValueError(
                f"TensorParallelPlan.degree={plan.degree} does not match topology.tp={self.topology.tp}"
            )
        plan.validate(hidden_size=getattr(getattr(module, "config", None), "hidden_size", None))
        return plan

    def _maybe_apply_tensor_parallel(self, module: torch.nn.Module) -> torch.nn.Module:
        if not self.topology.tp_enabled:
            return module
        plan = self._resolve_tensor_parallel_plan(module)
        module = apply_tensor_parallel(
            module, self._groups.get("tp"), plan, tp_rank=self.topology.tp_rank,
            tp_world=self.topology.tp,
        )
        if (plan.sequence_parallel and self.config.fused_collectives
                and self._device.type == "cuda" and self.topology.tp <= 8):
            # Sequence-parallel layout with the collectives inside the GEMMs: between the
            # parallel regions every tensor-parallel rank keeps B / tp whole sequences (the
            # dataloader wrapper hands each rank its slice), the column-parallel projections
            # gather them and the row-parallel ones scatter the sums back.
            from ohara_b200.parallel.tp_fused import LazyTPWorkspace

            width = int(getattr(getattr(module, "config", None), "hidden_size", 0)) or max(
                p.shape[-1] for p in module.parameters() if p.dim() == 2)
            attach_fused_workspace(module, LazyTPWorkspace(self._groups.get("tp"), width))
            self._tp_batch_sharding = True
            self._tp_grads_synced = True
        elif plan.sequence_parallel:
            # The same layout over the process group's all-gather / reduce-scatter (CPU ranks, or
            # fused collectives switched off): every tensor-parallel rank still keeps only its
            # B / tp sequences between the parallel regions.
            self._tp_batch_sharding = True
            self._tp_grads_synced = True
        elif (self.config.fused_collectives and self._device.type == "cuda"
              and self.topology.tp <= 16 and dist.get_backend() == Backend.NCCL.value):
            # Plain tensor parallelism: the all-reduce that ends a row-parallel layer runs as a
            # one-shot peer-memory kernel when the message is small (decode steps).
            from ohara_b200.parallel.peer import PeerRuntime

            attach_peer_runtime(module, PeerRuntime(self._groups.get("tp")))
        return module

    def local_batch(self, batch: Any) -> Any:
        """With sequence-parallel tensor parallelism each rank of a tensor-parallel group works
        on its own slice of the group's batch between the parallel regions: take that slice of
        every tensor of ``batch`` (dim 0). Otherwise the batch is returned unchanged."""
        by_batch = getattr(self, "_tp_batch_sharding", False)
        by_sequence = getattr(self, "_cp_sequence_sharding", False)
        if not (by_batch or by_sequence):
            return batch
        if isinstance(batch, torch.Tensor):
            if by_sequence and batch.dim() >= 2:
                from ohara_b200.parallel.cp import shard_sequence

                # zig-zag: an early and a late block per rank, equal attention work on every rank
                batch = shard_sequence(batch, self.topology.cp_rank, self.topology.cp, dim=1)
            if not by_batch or batch.dim() == 0:
                return batch
            tp, rank = self.topology.tp, self.topology.tp_rank
            if batch.shape[0] % tp:
                raise ValueError(f"batch of {batch.shape[0]} does not split over tp={tp}")
            per = batch.shape[0] // tp
            return batch[rank * per : (rank + 1) * per]
        if isinstance(batch, dict):
            return {k: self.local_batch(v) for k, v in batch.items()}
        if isinstance(batch, (tuple, list)):
            return type(batch)(self.local_batch(v) for v in batch)
        return batch

    def sync_tensor_parallel_gradients(self, model: torch.nn.Module) -> None:
        """Under the sequence-parallel layout the ranks of a tensor-parallel group see different
        tokens, so parameters that are *not* sharded (norms, embeddings, output head, routers)
        hold partial gradients: sum them over the group. Sharded parameters are already complete,
        their backward collectives mixed every rank's tokens in."""
        if not getattr(self, "_tp_batch_sharding", False) or self._tp_grads_synced:
            self.sync_context_parallel_gradients(model)
            return
        group = self._groups.get("tp")
        for param in model.parameters():
            if param.grad is not None and not hasattr(param, "tensor_parallel_dim"):
                dist.all_reduce(param.grad, group=group)
        self._tp_grads_synced = True
        self.sync_context_parallel_gradients(model)

    def sync_context_parallel_gradients(self, model: torch.nn.Module) -> None:
        """Context-parallel ranks see different tokens of the same sequences and no parameter is
        sharded between them: sum every gradient over the group."""
        if not getattr(self, "_cp_sequence_sharding", False) or self._replica_grads_synced:
            return
        if getattr(self, "_sharded_over_cp", False):
            return  # the sharded optimizer's group contains the context-parallel peers
        group = self._groups.get("cp")
        for param in model.parameters():
            if param.grad is not None:
                dist.all_reduce(param.grad, group=group)
        self._replica_grads_synced = True

    # -- data ----------------------------------------------------------------------------------
    def _replace_sampler(self, dataloader: DataLoader) -> DataLoader:
        dataset = getattr(dataloader, "dataset", None)
        if dataset is None or isinstance(dataset, IterableDataset):
            return dataloader
        if isinstance(getattr(dataloader, "sampler", None), DistributedSampler):
            return dataloader
        if dataloader.batch_size is None:
            return dataloader
        sampler = DistributedSampler(
            dataset, num_replicas=self._dp_world_size, rank=self._dp_rank,
            shuffle=isinstance(dataloader.sampler, RandomSampler), drop_last=dataloader.drop_last,
        )
        kwargs: dict[str, Any] = dict(
            dataset=dataset, batch_size=dataloader.batch_size, sampler=sampler,
            num_workers=dataloader.num_workers, collate_fn=dataloader.collate_fn,
            pin_memory=dataloader.pin_memory, drop_last=dataloader.drop_last,
            timeout=dataloader.timeout, worker_init_fn=dataloader.worker_init_fn,
            persistent_workers=dataloader.persistent_workers,
        )
        if dataloader.num_workers > 0:
            kwargs["prefetch_factor"] = dataloader.prefetch_factor
        return DataLoader(**kwargs)

    def prepare_dataloaders(self, *dataloaders: DataLoader):
        self.launch()
        if not dataloaders:
            raise ValueError("At least one dataloader is required")
        loaders = [
            self._replace_sampler(dl) if self._dp_world_size > 1 else dl for dl in dataloaders
        ]
        wrapped = [
            dl if isinstance(dl, _DeviceDataLoader) else _DeviceDataLoader(dl, self)
            for dl in loaders
        ]
        return tuple(wrapped) if len(wrapped) > 1 else wrapped[0]

    def to_device(self, value: Any) -> Any:
        """Recursively move the tensors of a nested batch to the compute device. CPU tensors going
        to a CUDA device are staged through pinned memory so the copy is asynchronous."""
        if isinstance(value, torch.Tensor):
            if value.device == self._device:
                return value
            if self._device.type == "cuda" and value.device.type == "cpu":
                if not value.is_pinned():
                    value = value.pin_memory()
                return value.to(self._device, non_blocking=True)
            return value.to(self._device)
        if isinstance(value, Mapping):
            moved = {key: self.to_device(item) for key, item in value.items()}
            try:
                return type(value)(moved)
            except TypeError:
                return moved
        if isinstance(value, tuple) and hasattr(value, "_fields"):
            return type(value)(*(self.to_device(item) for item in value))
        if isinstance(value, tuple):
            return tuple(self.to_device(item) for item in value)
        if isinstance(value, list):
            return [self.to_device(item) for item in value]
        return value

    # -- step helpers --------------------------------------------------------------------------
    def autocast_context(self):
        mode = self.config.precision.mode
        if self._device.type != "cuda":
            return nullcontext()
        if mode == PrecisionMode.FP16_MIXED:
            return torch.autocast(device_type="cuda", dtype=torch.float16)
        if mode == PrecisionMode.BF16_MIXED:
            return torch.autocast(device_type="cuda", dtype=torch.bfloat16)
        return nullcontext()

    def backward(self, loss: torch.Tensor) -> None:
        if getattr(self, "_tp_batch_sharding", False):
            # every rank's loss is a mean over its own slice: the group mean is their average
            loss = loss / self.topology.tp
            self._tp_grads_synced = False
        if getattr(self, "_cp_sequence_sharding", False) and not getattr(self, "_sharded_over_cp", False):
            # (under the sharded optimizer the reduce-scatter takes the mean over the
            # context-parallel peers as well, so the loss keeps its scale)
            loss = loss / self.topology.cp
            self._replica_grads_synced = False
        if self._scaler.is_enabled():
            self._scaler.scale(loss).backward()
        else:
            loss.backward()
        sharding = getattr(getattr(self, "_module", None), "_param_sharding", None)
        if sharding is not None:
            sharding.finish_backward()  # units whose gradients did not all arrive

    def no_sync(self, module: torch.nn.Module, enabled: bool = True):
        return self._strategy.no_sync(module, enabled=enabled)

    def no_backward_sync(self, module: torch.nn.Module, enabled: bool = True):
        return self.no_sync(module, enabled=enabled)

    def clip_gradients(self, model: torch.nn.Module, optimizer: Optimizer, max_norm: float) -> torch.Tensor:
        if self._scaler.is_enabled():
            self._scaler.unscale_(optimizer)
        self.sync_tensor_parallel_gradients(model)
        self.sync_expert_gradients(model)
        clip = getattr(optimizer, "clip_grad_norm_", None)
        if callable(clip):  # sharded optimizers know how to form the global norm
            return clip(model, max_norm)
        if self.launched and (self.topology.tp_enabled or self.topology.ep > 1
                              or self.topology.pp > 1):
            return self._clip_sharded(model, max_norm)
        return torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=max_norm)

    def _clip_sharded(self, model: torch.nn.Module, max_norm: float) -> torch.Tensor:
        """Global gradient norm when parameters are sharded: squared norms of tensor-parallel
        shards are summed over the ``tp`` group, those of expert shards over the ``ep`` group,
        replicated parameters are counted once; every rank then applies the same coefficient."""
        zero = torch.zeros((), device=self._device)
        parts = {"tp": zero.clone(), "ep": zero.clone(), "whole": zero.clone()}
        grads = []
        for p in model.parameters():
            if p.grad is None:
                continue
            kind = ("tp" if hasattr(p, "tensor_parallel_dim")
                    else "ep" if getattr(p, "expert_parallel", False) else "whole")
            parts[kind] = parts[kind] + p.grad.float().square().sum()
            grads.append(p.grad)
        if not grads:
            return zero
        if self.topology.tp_enabled:
            dist.all_reduce(parts["tp"], group=self._groups.get("tp"))
        if self.topology.ep > 1:
            dist.all_reduce(parts["ep"], group=self._groups.get("ep"))
        total = parts["tp"] + parts["ep"] + parts["whole"]
        if self.topology.pp > 1:  # every pipeline stage holds different parameters
            dist.all_reduce(total, group=self._groups.get("pp"))
        total = total.sqrt()
        scale = (max_norm / (total + 1e-6)).clamp(max=1.0)
        for grad in grads:
            grad.mul_(scale.to(grad.dtype))
        return total

    def optimizer_step(self, optimizer: Optimizer) -> None:
        module = getattr(self, "_module", None)
        if module is not None:
            self.sync_tensor_parallel_gradients(module)
            self.sync_expert_gradients(module)
        if self._scaler.is_enabled():
            self._scaler.step(optimizer)
            self._scaler.update()
        else:
            optimizer.step()

    # -- collectives ---------------------------------------------------------------------------
    def barrier(self) -> None:
        if dist.is_initialized():
            if dist.get_backend() == Backend.NCCL.value and self._device.type == "cuda":
                dist.barrier(device_ids=[self._device.index])
            else:
                dist.barrier()

    def synchronize(self) -> None:
        if self._device.type == "cuda":
            torch.cuda.synchronize(self._device)

    def broadcast(self, obj: Any, src: int = 0) -> Any:
        if not dist.is_initialized():
            return obj
        payload = [obj]
        dist.broadcast_object_list(payload, src=src)
        return payload[0]

    def all_reduce(self, tensor: torch.Tensor, reduce_type: ReduceType | str = ReduceType.MEAN, *,
                   group: Any | None = None, reduce_op: ReduceType | str | None = None) -> torch.Tensor:
        selected = reduce_op if reduce_op is not None else reduce_type
        if isinstance(selected, str):
            selected = ReduceType(selected)
        if selected not in _REDUCE_OPS:
            raise ValueError(f"Unsupported reduce type: {selected}")
        if not dist.is_initialized():
            return tensor
        dist.all_reduce(tensor, op=getattr(dist.ReduceOp, _REDUCE_OPS[selected]), group=group)
        if selected == ReduceType.MEAN:
            tensor /= dist.get_world_size(group=group) if group is not None else self.world_size
        return tensor

    def all_gather(self, tensor: torch.Tensor, group: Any | None = None) -> list[torch.Tensor]:
        if not dist.is_initialized():
            return [tensor]
        world = dist.get_world_size(group=group) if group is not None else self.world_size
        gathered = [torch.zeros_like(tensor) for _ in range(world)]
        dist.all_gather(gathered, tensor, group=group)
        return gathered

    # -- checkpoints ---------------------------------------------------------------------------
    def full_state_dict(self, module: torch.nn.Module) -> dict[str, torch.Tensor]:
        """Unsharded, wrapper-free state dict of ``module`` (collective when TP/FSDP is active):
        what the reference's ``Llama`` can load directly."""
        inner = module.module if hasattr(module, "module") else module
        sharding = getattr(inner, "_param_sharding", None)
        if sharding is not None:
            if not self.topology.tp_enabled:
                return sharding.full_state_dict(inner)
            with sharding.gathered():  # whole tensor shards first, then whole matrices
                return {k: v.detach().clone() for k, v in gather_tensor_parallel_state(
                    inner, self._groups.get("tp")).items()}
        sync = getattr(getattr(self, "_sharded_optimizer", None), "sync_master_weights", None)
        if callable(sync):
            sync()
        stage = getattr(inner, "stage", None) if getattr(inner, "pipeline_stage", False) else None
        source = stage if stage is not None else inner
        if self.topology.tp_enabled:
            state = gather_tensor_parallel_state(source, self._groups.get("tp"))
        else:
            state = dict(source.state_dict())
        if stage is not None:
            return self._gather_pipeline_state(stage, state)
        if getattr(self, "_expert_parallel", False):
            # routed experts: every rank of the expert-parallel group holds E / ep of them
            group, world = self._groups.get("ep"), self.topology.ep
            for name, param in inner.named_parameters():
                if getattr(param, "expert_parallel", False) and name in state:
                    parts = [torch.empty_like(state[name]) for _ in range(world)]
                    dist.all_gather(parts, state[name].contiguous(), group=group)
                    state[name] = torch.cat(parts, dim=0)
        return state

    def save(self, path: str | Path, state: dict[str, Any]) -> None:
        """Rank 0 writes ``state`` atomically (temp file + rename), then everyone meets at a
        barrier. Collective state (sharded optimizers) must be materialised by the caller."""
        path = Path(path)
        if self.is_global_zero:
            path.parent.mkdir(parents=True, exist_ok=True)
            temporary = path.with_name(f".{path.name}.tmp-{os.getpid()}")
            try:
                torch.save(state, temporary)
                os.replace(temporary, path)
            finally:
                temporary.unlink(missing_ok=True)
        self.barrier()

    def load(self, path: str | Path, state: dict[str, Any] | None = None) -> dict[str, Any]:
        try:
            payload: dict[str, Any] = torch.load(Path(path), map_location=self._device,
                                                 weights_only=False)
        except FileNotFoundError:
            raise
        except Exception as error:  # noqa: BLE001 - a damaged file surfaces as many different errors
            # (zip, pickle, EOF ...): name the file, keep the cause. ``save`` never leaves such a
            # file behind (it renames a complete temporary file), so this is damage from outside.
            from ohara_b200.errors import CheckpointError

            raise CheckpointError(f"{path} is not a readable checkpoint "
                                  f"({type(error).__name__}: {error})") from error
        if not isinstance(payload, dict):
            from ohara_b200.errors import CheckpointError

            raise CheckpointError(f"{path} holds a {type(payload).__name__}, not a checkpoint")
        if state is None:
            return payload
        for key, obj in state.items():
            if key not in payload:
                continue
            sharding = getattr(obj.module if hasattr(obj, "module") else obj, "_param_sharding", None)
            if isinstance(obj, torch.nn.Module):
                # checkpoints hold whole tensors (``full_state_dict``): cut out what this rank
                # keeps of tensor-parallel matrices and expert stacks
                # wrapper-free keys, whatever wrote the file (a DDP- or torch.compile-wrapped
                # module prefixes its keys, as the reference's checkpoints do)
                saved = {_strip_wrapper_prefixes(name): tensor
                         for name, tensor in payload[key].items()}
                inner = obj.module if hasattr(obj, "module") else obj
                local = self._local_slice_of_state(inner, saved)
                if sharding is not None:  # parameters sharded per block: load through the gather
                    sharding.load_full_state_dict(inner, local)
                elif getattr(inner, "pipeline_stage", False):
                    inner.stage.load_state_dict(local)
                else:
                    inner.load_state_dict(local)
            elif hasattr(obj, "load_state_dict"):
                saved = payload[key]
                if isinstance(saved, dict) and saved.get("model_parallel"):
                    topo = self.topology
                    layout = (saved["tp"], saved["ep"], saved.get("pp", 1))
                    if layout != (topo.tp, topo.ep, topo.pp):
                        raise ValueError(
                            f"optimizer state of a (tp, ep, pp) = {layout} run cannot be loaded "
                            f"into (tp, ep, pp) = {(topo.tp, topo.ep, topo.pp)}")
                    saved = saved["states"][(topo.tp_rank, topo.ep_rank, topo.pp_rank)]
                obj.load_state_dict(saved)
            else:
                state[key] = payload[key]
        return payload

    def _gather_pipeline_state(self, stage, state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """Whole-model state dict from the stages' ones (collective over the pipeline group):
        block indices become the model's own, the embedding comes from the first stage, the final
        norm and the output projection from the last, the rotary tables from this stage."""
        begin, _ = stage.layer_range
        renamed = {}
        for name, tensor in state.items():
            renamed[_stage_to_model_name(name, begin)] = tensor.detach().cpu()
        parts: list[Any] = [None] * self.topology.pp
        dist.all_gather_object(parts, renamed, group=self._groups.get("pp"))
        merged: dict[str, torch.Tensor] = {}
        for part in parts:
            merged.update(part)
        merged["freq_cos"] = stage.freq_cos.detach().cpu()
        merged["freq_sin"] = stage.freq_sin.detach().cpu()
        return merged

    def optimizer_state_dict(self, optimizer: Optimizer) -> dict[str, Any]:
        """``optimizer.state_dict()`` for a checkpoint that one rank writes (collective). Ranks
        with different tensor-parallel or expert-parallel coordinates hold optimizer state for
        different shards, so their states are collected, one per coordinate (from the first
        data-parallel replica of each); :meth:`load` hands every rank its own again."""
        state = optimizer.state_dict()
        topo = self.topology
        if not self.launched or not (topo.tp_enabled or topo.ep > 1 or topo.pp > 1):
            return state
        mine = (topo.tp_rank, topo.ep_rank, topo.pp_rank)
        first_replica = topo.dp_rank == 0 and topo.cp_rank == 0
        # only the rank that writes the file collects the states: with all-gather every rank would
        # hold the optimizer state of the whole model in host memory
        writer = self.is_global_zero
        gathered: list[Any] | None = [None] * topo.world_size if writer else None
        dist.gather_object((mine, state if first_replica else None), gathered, dst=0)
        states = ({coordinate: entry for coordinate, entry in gathered if entry is not None}
                  if writer else {mine: state})
        return {"model_parallel": True, "tp": topo.tp, "ep": topo.ep, "pp": topo.pp,
                "states": states}

    def _local_slice_of_state(self, module: torch.nn.Module,
                              state: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        """The inverse of :meth:`full_state_dict` for one rank: tensor-parallel parameters keep
        their ``1 / tp`` slice along the sharded dimension, expert-parallel stacks their
        ``E / ep`` experts; everything else is passed through. Tensors that already have the
        local shape are left alone, so a state dict saved from a sharded module loads too."""
        inner = module.module if hasattr(module, "module") else module
        topo = self.topology
        if getattr(inner, "pipeline_stage", False):
            # keep what this stage holds, under the stage's own (local) block indices
            stage = inner.stage
            begin, _ = stage.layer_range
            wanted = {_stage_to_model_name(name, begin): name for name in stage.state_dict()}
            state = {wanted[name]: tensor for name, tensor in state.items() if name in wanted}
            inner = stage
        if not (topo.tp_enabled or getattr(self, "_expert_parallel", False)):
            return state
        local = dict(state)
        for name, param in inner.named_parameters():
            tensor = state.get(name)
            if tensor is None or tuple(tensor.shape) == tuple(param.shape):
                continue
            dim = getattr(param, "tensor_parallel_dim", None)
            if dim is not None and tensor.shape[dim] == param.shape[dim] * topo.tp:
                width = param.shape[dim]
                tensor = tensor.narrow(dim, topo.tp_rank * width, width)
            if getattr(param, "expert_parallel", False) and tensor.shape[0] == param.shape[0] * topo.ep:
                count = param.shape[0]
                tensor = tensor.narrow(0, topo.ep_rank * count, count)
            local[name] = tensor
        return local

    def log_dict(self, payload: dict[str, Any], step: int | None = None) -> None:
        if not self.is_global_zero:
            return
        for logger in self.loggers:
            if hasattr(logger, "log_metrics"):
                logger.log_metrics(payload, step=step)
            elif hasattr(logger, "log_dict"):
                logger.log_dict(payload, step=step)

    def close(self) -> None:
        if self.heartbeat is not None:
            self.heartbeat.stop()
            self.heartbeat = None
        if self.watchdog is not None:
            self.watchdog.close()
            self.watchdog = None
        if dist.is_initialized():
            dist.destroy_process_group()
