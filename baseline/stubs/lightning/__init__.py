"""Minimal stand-in for the ``lightning`` package, used only by the reference-arm harness.

The reference imports ``lightning`` at ``import ohara.utils`` time for a parameter-count summary
(ohara/utils/info.py:2-4). ``lightning`` is not installed on this image and cannot be fetched, so
the harness puts this stub on ``sys.path``; none of it is on the timed path.
"""

import torch.nn as nn


class LightningModule(nn.Module):
    pass


class Fabric:  # pragma: no cover - never instantiated by the harness
    def __init__(self, *args, **kwargs):
        raise RuntimeError("lightning.Fabric is not available in this environment")
