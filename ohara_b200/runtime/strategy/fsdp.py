"""Sharded data parallelism: the module stays a plain ``nn.Module`` (no wrapper, no prefixed
state-dict keys); the optimizer is wrapped by :class:`ohara_b200.parallel.zero.ShardedOptimizer`,
which owns the gradient reduce-scatter, the sharded master weights / optimizer state and the
parameter all-gather. See ``ohara_b200/parallel/zero.py`` for the data layout. With
``shard_parameters=True`` the parameters themselves are sharded per transformer block
(``ohara_b200/parallel/param_shard.py``) and the optimizer runs on the master shards.

The engine tells the strategy which process groups to use (:meth:`FSDPStrategy.configure`):

* ``process_group``: the ranks the dense parameters are sharded over (``dp_shard``, together with
  the context-parallel and expert-parallel peers, which are replicas as far as dense parameters
  are concerned);
* ``replicate_group``: with hybrid sharding (``dp_replicate > 1`` and ``dp_shard > 1``) the ranks
  that hold the same shard; their reduced gradients are averaged;
* ``expert_group``: with expert parallelism, the ranks that hold the same routed experts; the
  expert parameters form a second part of the optimizer sharded over those ranks only;
* ``norm_groups``: the tensor- / expert-parallel groups, over which a global gradient norm has to
  add up the distinct shards.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from .base import BaseStrategy


class FSDPStrategy(BaseStrategy):
    name = "fsdp"

    def __init__(self, *, fused: bool = True, init_sync: bool = True,
                 shard_parameters: bool = False, shard_parameters_layout: str = "even") -> None:
        self.fused = fused
        self.init_sync = init_sync
        self.shard_parameters = shard_parameters
        self.shard_parameters_layout = shard_parameters_layout
        self.process_group = None
        self.device: torch.device | None = None
        self.replicate_group = None
        self.replicate_world = 1
        self.expert_parallel = False
        self.expert_group = None
        self.expert_world = 1
        self.norm_groups: dict[str, Any] = {}
        self.shard_world: int | None = None

    @property
    def solo(self) -> bool:
        return self.shard_world is not None and self.shard_world <= 1

    def configure(self, *, replicate_group=None, replicate_world: int = 1,
                  expert_parallel: bool = False, expert_group=None, expert_world: int = 1,
                  norm_groups: dict[str, Any] | None = None, shard_world: int | None = None) -> None:
        """``shard_world``: size of the group the dense parameters are sharded over. When it is 1
        although the job has several ranks (all of them tensor-parallel peers, say) the optimizer
        shards over nobody: falling back to the default group would mix different tensor shards."""
        self.shard_world = shard_world
        self.replicate_group, self.replicate_world = replicate_group, replicate_world
        self.expert_parallel = expert_parallel
        self.expert_group, self.expert_world = expert_group, expert_world
        self.norm_groups = dict(norm_groups or {})

    def setup_module(self, module: nn.Module, *, device: torch.device,
                     process_group: Any | None = None) -> nn.Module:
        import torch.distributed as dist

        self.process_group = process_group
        self.device = device
        if self.init_sync and dist.is_initialized() and not self.solo:
            # Replicas must start from identical weights, as DDP guarantees.
            src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
            for tensor in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(tensor.data, src=src, group=process_group)
        if self.shard_parameters:
            from ohara_b200.parallel.param_shard import shard_llama

            shard_llama(module, process_group, solo=self.solo,
                        replicate_group=self.replicate_group,
                        replicate_world=self.replicate_world,
                        layout=self.shard_parameters_layout)
        return module

    def setup_optimizer(self, optimizer, module: nn.Module | None = None):
        from ohara_b200.parallel.zero import HybridShardedOptimizer, ShardedOptimizer

        if isinstance(optimizer, (ShardedOptimizer, HybridShardedOptimizer)):
            return optimizer
        sharding = getattr(module, "_param_sharding", None)
        if sharding is not None:
            from ohara_b200.parallel.param_shard import ParameterShardedOptimizer

            if isinstance(optimizer, ParameterShardedOptimizer):
                return optimizer
            return ParameterShardedOptimizer(
                optimizer, sharding,
                norm_groups={k: v for k, v in self.norm_groups.items() if k == "tp"})
        dense_norms = {k: v for k, v in self.norm_groups.items() if k in ("tp", "pp")}
        common = dict(fused=self.fused, replicate_group=self.replicate_group,
                      replicate_world=self.replicate_world)
        if not self.expert_parallel:
            return ShardedOptimizer(optimizer, process_group=self.process_group,
                                    norm_groups=dense_norms, solo=self.solo, **common)

        def is_expert(p) -> bool:
            return bool(getattr(p, "expert_parallel", False))

        return HybridShardedOptimizer(optimizer, [
            dict(select=lambda p: not is_expert(p), process_group=self.process_group,
                 norm_groups=dense_norms, solo=self.solo, **common),
            dict(select=is_expert, process_group=self.expert_group,
                 solo=self.expert_world <= 1, norm_groups=self.norm_groups, **common),
        ])
