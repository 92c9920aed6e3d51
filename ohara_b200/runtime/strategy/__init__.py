from .base import BaseStrategy
from .ddp import DDPStrategy
from .fsdp import FSDPStrategy
from .single import SingleStrategy

__all__ = ["BaseStrategy", "DDPStrategy", "FSDPStrategy", "SingleStrategy"]
