from .info import model_summary  # noqa: F401
from .rand import random_name  # noqa: F401
from .svd import svd_approx  # noqa: F401
from .tools import BetterCycle, auto_accelerator, build_mask  # noqa: F401
