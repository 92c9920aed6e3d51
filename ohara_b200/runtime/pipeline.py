"""Pipeline-parallel plan description (reference: ohara/runtime/pipeline.py:8-32)."""

from __future__ import annotations

from dataclasses import dataclass, field

from .enums import PipelineScheduleType


@dataclass
class PipelineStageSpec:
    module_names: list[str]


@dataclass
class PipelinePlan:
    degree: int = 1
    micro_batch_size: int = 1
    schedule: PipelineScheduleType = PipelineScheduleType.ONE_FWD_ONE_BWD
    stages: list[PipelineStageSpec] = field(default_factory=list)

    def validate(self, local_batch_size: int) -> None:
        if self.degree < 1:
            raise ValueError("pipeline degree must be >= 1")
        if self.micro_batch_size < 1:
            raise ValueError("pipeline micro_batch_size must be >= 1")
        if local_batch_size % self.micro_batch_size != 0:
            raise ValueError(
                f"local_batch_size={local_batch_size} must be divisible by "
                f"micro_batch_size={self.micro_batch_size}"
            )
        if self.stages and len(self.stages) % self.degree != 0:
            raise ValueError(
                f"number of virtual stages={len(self.stages)} must be divisible by pipeline "
                f"degree={self.degree}"
            )

    def stages_for_rank(self, pp_rank: int) -> list[PipelineStageSpec]:
        """Virtual stages owned by ``pp_rank`` under an interleaved (round-robin) assignment."""
        return [stage for idx, stage in enumerate(self.stages) if idx % self.degree == pp_rank]
