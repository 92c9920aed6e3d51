from .config import (
    DistributedConfig,
    EngineConfig,
    FaultToleranceConfig,
    ParallelConfig,
    PrecisionConfig,
)
from .engine import OharaEngine
from .enums import (
    Backend,
    ParallelDimension,
    PipelineScheduleType,
    PrecisionMode,
    ReduceType,
    StrategyType,
    TensorParallelStyle,
)
from .pipeline import PipelinePlan, PipelineStageSpec
from .tensor_parallel import TensorParallelPlan, TensorParallelRule
from .topology import ParallelTopology
from .watchdog import CollectiveTimeout, Heartbeat, PeerFailure, StepWatchdog

__all__ = [
    "Backend",
    "CollectiveTimeout",
    "DistributedConfig",
    "EngineConfig",
    "FaultToleranceConfig",
    "Heartbeat",
    "OharaEngine",
    "ParallelConfig",
    "ParallelDimension",
    "ParallelTopology",
    "PeerFailure",
    "PipelinePlan",
    "PipelineScheduleType",
    "PipelineStageSpec",
    "PrecisionConfig",
    "PrecisionMode",
    "ReduceType",
    "StepWatchdog",
    "StrategyType",
    "TensorParallelPlan",
    "TensorParallelRule",
    "TensorParallelStyle",
]
