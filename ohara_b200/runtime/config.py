"""Dataclass configuration of the engine (reference: ohara/runtime/config.py:9-37)."""

from __future__ import annotations

from dataclasses import dataclass, field

from .enums import Backend, PrecisionMode, StrategyType
from .pipeline import PipelinePlan
from .tensor_parallel import TensorParallelPlan


@dataclass
class DistributedConfig:
    backend: Backend = Backend.NCCL
    timeout_seconds: int = 1800


@dataclass
class ParallelConfig:
    dp_replicate: int = 1
    dp_shard: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    infer_dp_shard_from_world_size: bool = True


@dataclass
class PrecisionConfig:
    mode: PrecisionMode = PrecisionMode.BF16_MIXED


@dataclass
class FaultToleranceConfig:
    """Host-side failure detection (all off by default, like the reference, whose only detector is
    the process-group timeout). ``heartbeat_interval_s > 0`` starts a heartbeat thread per rank
    over the rendezvous store; ``step_timeout_s > 0`` arms a deadline around every guarded step."""

    heartbeat_interval_s: float = 0.0
    heartbeat_timeout_s: float = 30.0
    step_timeout_s: float = 0.0
    exit_on_step_timeout: bool = False


@dataclass
class EngineConfig:
    strategy: StrategyType = StrategyType.AUTO
    distributed: DistributedConfig = field(default_factory=DistributedConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    precision: PrecisionConfig = field(default_factory=PrecisionConfig)
    tensor_parallel: TensorParallelPlan = field(default_factory=TensorParallelPlan)
    fault_tolerance: FaultToleranceConfig = field(default_factory=FaultToleranceConfig)
    # Pipeline parallelism (``parallel.pp > 1``): sequences per pipeline micro-batch.
    pipeline: PipelinePlan = field(default_factory=PipelinePlan)
    # Use the peer-memory (NVLink) fused collectives where available; False keeps every
    # collective on the c10d backend (the A/B baseline and the only choice on CPU/gloo).
    fused_collectives: bool = True
    # Expert parallelism: rows a rank can receive for its experts in one layer, as a multiple of
    # its fair share; pairs beyond it are dropped.
    expert_capacity_factor: float = 2.0
    # Recompute every transformer block in the backward pass instead of keeping its activations
    # (models that offer ``enable_activation_checkpointing``).
    activation_checkpointing: bool = False
    # How attention sees the whole sequence under context parallelism (cp > 1): "ring" exchanges
    # keys / values over NVLink peer memory under the flash kernels; "ulysses" re-partitions
    # q / k / v from sequence shards to head shards with all-to-alls (needs heads >= cp).
    context_parallel_mode: str = "ring"
    # StrategyType.FSDP only: shard the parameters themselves per transformer block (gathered
    # just before a block runs, released after it) instead of the optimizer state alone.
    shard_parameters: bool = False
    # "even": equal ranges (AdamW); "matrix": every matrix of a block whole at one owner (Muon)
    shard_parameters_layout: str = "even"
