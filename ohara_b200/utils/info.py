"""Parameter-count summary of a module, with no dependency beyond torch
(the reference delegates to lightning's ModelSummary: ohara/utils/info.py:7-46)."""

from __future__ import annotations

import torch.nn as nn


def convert_int_to_shortened_string(num: int) -> str:
    """1234 -> '1.2K', 5_600_000 -> '5.6M', and so on up to trillions."""
    for limit, suffix in ((1e3, ""), (1e6, "K"), (1e9, "M"), (1e12, "B")):
        if abs(num) < limit:
            return str(num) if not suffix else f"{num / (limit / 1e3):.1f}{suffix}"
    return f"{num / 1e12:.1f}T"


class Summary:
    """Per-top-level-child parameter table; ``str()`` renders it."""

    def __init__(self, model: nn.Module) -> None:
        self.rows = [
            (name, type(child).__name__, sum(p.numel() for p in child.parameters()))
            for name, child in model.named_children()
        ]
        params = list(model.parameters())
        self.total_parameters = sum(p.numel() for p in params)
        self.trainable_parameters = sum(p.numel() for p in params if p.requires_grad)

    def __str__(self) -> str:
        lines = [f"{'name':<24}{'type':<24}{'params':>12}"]
        lines += [f"{n:<24}{t:<24}{convert_int_to_shortened_string(c):>12}" for n, t, c in self.rows]
        lines.append(f"total {convert_int_to_shortened_string(self.total_parameters)}, "
                     f"trainable {convert_int_to_shortened_string(self.trainable_parameters)}")
        return "\n".join(lines)


class Model(nn.Module):
    """A module that only holds ``model``. The reference wraps models in a Lightning module of
    this name to reuse Lightning's summary (ohara/utils/info.py:7-10); there is no Lightning
    here, the class is kept for callers that construct it."""

    def __init__(self, model: nn.Module, *args, **kwargs) -> None:
        super().__init__()
        self.model = model

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)


def model_summary(model: nn.Module, print_summary: bool = False) -> dict:
    summary = Summary(model)
    if print_summary:
        print(summary)
    return {
        "summary": summary,
        "total_parameters": convert_int_to_shortened_string(summary.total_parameters),
        "trainable_parameters": convert_int_to_shortened_string(summary.trainable_parameters),
    }
