from .config import DistributedConfig, EngineConfig, ParallelConfig, PrecisionConfig
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

__all__ = [
    "Backend",
    "DistributedConfig",
    "EngineConfig",
    "OharaEngine",
    "ParallelConfig",
    "ParallelDimension",
    "ParallelTopology",
    "PipelinePlan",
    "PipelineScheduleType",
    "PipelineStageSpec",
    "PrecisionConfig",
    "PrecisionMode",
    "ReduceType",
    "StrategyType",
    "TensorParallelPlan",
    "TensorParallelRule",
    "TensorParallelStyle",
]
