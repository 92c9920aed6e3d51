"""String enums of the runtime configuration (reference: ohara/runtime/enums.py:6-48).

``StrategyType.FSDP`` and ``TensorParallelStyle.SEQUENCE`` do not exist in the reference: the first
selects the sharded-optimizer data-parallel strategy of this package, the second marks modules
that run on sequence shards between tensor-parallel regions.
"""

from __future__ import annotations

from enum import StrEnum


class Backend(StrEnum):
    NCCL = "nccl"
    GLOO = "gloo"
    MPI = "mpi"


class StrategyType(StrEnum):
    AUTO = "auto"
    SINGLE = "single"
    DDP = "ddp"
    FSDP = "fsdp"


class PrecisionMode(StrEnum):
    FP32 = "fp32"
    FP16_MIXED = "fp16_mixed"
    BF16_MIXED = "bf16_mixed"
    BF16_TRUE = "bf16_true"


class ReduceType(StrEnum):
    SUM = "sum"
    MEAN = "mean"
    MAX = "max"
    MIN = "min"


class PipelineScheduleType(StrEnum):
    ONE_FWD_ONE_BWD = "1f1b"
    GPIPE = "gpipe"


class ParallelDimension(StrEnum):
    DP_REPLICATE = "dp_replicate"
    DP_SHARD = "dp_shard"
    TP = "tp"
    PP = "pp"
    CP = "cp"
    EP = "ep"


class TensorParallelStyle(StrEnum):
    COLWISE = "colwise"
    ROWWISE = "rowwise"
    # column-parallel with the outputs of all ranks concatenated again (an output head whose
    # logits every rank needs in full)
    COLWISE_GATHERED = "colwise_gathered"
