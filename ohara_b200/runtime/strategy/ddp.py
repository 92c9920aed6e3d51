"""Replicated data parallelism through ``torch.nn.parallel.DistributedDataParallel`` — the
reference's only multi-process strategy (ohara/runtime/strategy/ddp.py:11-34), kept as the
fallback and as the A/B baseline for the sharded strategy."""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel

from .base import BaseStrategy


class DDPStrategy(BaseStrategy):
    name = "ddp"

    def __init__(self, *, init_sync: bool = True) -> None:
        self._init_sync = init_sync

    def setup_module(self, module: nn.Module, *, device: torch.device,
                     process_group: Any | None = None) -> nn.Module:
        kwargs: dict[str, Any] = {"process_group": process_group, "init_sync": self._init_sync}
        if device.type == "cuda":
            kwargs.update(device_ids=[device.index], output_device=device.index)
        return DistributedDataParallel(module, **kwargs)
