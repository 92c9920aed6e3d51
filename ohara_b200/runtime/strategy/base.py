"""Strategy interface: how a module is wrapped for data parallelism and how gradient
synchronisation is suppressed during accumulation (reference: ohara/runtime/strategy/base.py)."""

from __future__ import annotations

from contextlib import AbstractContextManager, nullcontext
from typing import Any

import torch
import torch.nn as nn


class BaseStrategy:
    name = "base"

    def setup_module(self, module: nn.Module, *, device: torch.device,
                     process_group: Any | None = None) -> nn.Module:
        raise NotImplementedError

    def setup_optimizer(self, optimizer, module: nn.Module | None = None):
        return optimizer

    def no_sync(self, module: nn.Module, enabled: bool):
        """Context that skips gradient synchronisation for the backward passes inside it."""
        if not enabled:
            return nullcontext()
        factory = getattr(module, "no_sync", None)
        if callable(factory):
            ctx = factory()
            if isinstance(ctx, AbstractContextManager):
                return ctx
        return nullcontext()
