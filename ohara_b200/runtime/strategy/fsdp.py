"""Sharded data parallelism: the module stays a plain ``nn.Module`` (no wrapper, no prefixed
state-dict keys); the optimizer is wrapped by :class:`ohara_b200.parallel.zero.ShardedOptimizer`,
which owns the gradient reduce-scatter, the sharded master weights / optimizer state and the
parameter all-gather. See ``ohara_b200/parallel/zero.py`` for the data layout."""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from .base import BaseStrategy


class FSDPStrategy(BaseStrategy):
    name = "fsdp"

    def __init__(self, *, fused: bool = True, init_sync: bool = True) -> None:
        self.fused = fused
        self.init_sync = init_sync
        self.process_group = None
        self.device: torch.device | None = None

    def setup_module(self, module: nn.Module, *, device: torch.device,
                     process_group: Any | None = None) -> nn.Module:
        import torch.distributed as dist

        self.process_group = process_group
        self.device = device
        if self.init_sync and dist.is_initialized():
            # Replicas must start from identical weights, as DDP guarantees.
            src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
            for tensor in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(tensor.data, src=src, group=process_group)
        return module

    def setup_optimizer(self, optimizer, module: nn.Module | None = None):
        from ohara_b200.parallel.zero import ShardedOptimizer

        if isinstance(optimizer, ShardedOptimizer):
            return optimizer
        return ShardedOptimizer(optimizer, process_group=self.process_group, fused=self.fused)
