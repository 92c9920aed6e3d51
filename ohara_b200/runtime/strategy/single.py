"""Single-process strategy: the module is used as is."""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from .base import BaseStrategy


class SingleStrategy(BaseStrategy):
    name = "single"

    def setup_module(self, module: nn.Module, *, device: torch.device,
                     process_group: Any | None = None) -> nn.Module:
        return module
