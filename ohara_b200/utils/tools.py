"""Small helpers: device selection, attention masks and a re-iterable infinite cycle
(reference: ohara/utils/tools.py:10-85)."""

from __future__ import annotations

from collections.abc import Iterable
from dataclasses import dataclass
from typing import Any

import torch


def auto_accelerator(device: str | torch.device | None = None) -> torch.device:
    """Return ``device`` if given, else the best available of cuda / mps / cpu."""
    if isinstance(device, torch.device):
        return device
    if isinstance(device, str):
        return torch.device(device)
    assert device is None, "Pass Valid Device"
    if torch.cuda.is_available():
        return torch.device("cuda")
    if torch.backends.mps.is_available():
        return torch.device("mps")
    return torch.device("cpu")


def build_mask(seq_len: int, sliding_window_attention: bool = False, window_size: int = 1):
    """Additive ``(1, 1, T, T)`` mask: 0 where key j is visible to query i (causal, optionally
    limited to the last ``window_size`` positions), ``-inf`` elsewhere."""
    assert window_size != 0, "window_size cannot be 0"
    if not sliding_window_attention:
        window_size = seq_len
    distance = torch.arange(seq_len).unsqueeze(-1) - torch.arange(seq_len)
    mask = torch.full((seq_len, seq_len), float("-inf"))
    mask[(distance >= 0) & (distance <= window_size - 1)] = 0
    return mask[None, None]


@dataclass
class BetterCycle:
    """Iterate over ``iterable`` forever, restarting it when exhausted; ``idx`` counts restarts."""

    iterable: Iterable
    idx: int = 0
    _iterator: Any = None

    def __iter__(self) -> "BetterCycle":
        return self

    def __next__(self) -> Any:
        if self._iterator is None:
            self._iterator = iter(self.iterable)
        try:
            return next(self._iterator)
        except StopIteration:
            self.idx += 1
            self._iterator = iter(self.iterable)
            return next(self._iterator)

    def close(self) -> None:
        """Drop the live iterator so generators and dataloader workers can shut down."""
        self._iterator = None
