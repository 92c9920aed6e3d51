"""Rank arithmetic for the six parallel dimensions.

Ranks are laid out (outermost to innermost) ``pp, dp_replicate, dp_shard, cp, tp, ep`` — the order
the reference uses (ohara/runtime/topology.py:85-101), which keeps tensor/expert-parallel peers on
neighbouring ranks. Everything here is pure integer arithmetic; process groups are created by the
engine from the rank lists this class produces.
"""

from __future__ import annotations

import os
from collections.abc import Iterable
from dataclasses import dataclass
from itertools import product

from .config import ParallelConfig

_ORDER = ("pp", "dp_replicate", "dp_shard", "cp", "tp", "ep")


@dataclass
class ParallelTopology:
    world_size: int
    dp_replicate: int
    dp_shard: int
    tp: int
    pp: int
    cp: int
    ep: int

    @classmethod
    def from_config(cls, world_size: int, config: ParallelConfig) -> "ParallelTopology":
        fixed = {name: int(getattr(config, name)) for name in _ORDER}
        base = fixed["dp_replicate"] * fixed["tp"] * fixed["pp"] * fixed["cp"] * fixed["ep"]
        if base < 1:
            raise ValueError("Invalid parallel dimensions: base product must be >= 1")
        if config.infer_dp_shard_from_world_size:
            if world_size % base != 0:
                raise ValueError(
                    f"world_size={world_size} is not divisible by dp_replicate*tp*pp*cp*ep={base}"
                )
            fixed["dp_shard"] = world_size // base
        return cls(world_size=world_size, **fixed)

    def __post_init__(self) -> None:
        sizes = self._sizes()
        if any(size < 1 for size in sizes):
            raise ValueError("All parallel dimensions must be >= 1")
        total = 1
        for size in sizes:
            total *= size
        if total != self.world_size:
            raise ValueError(
                f"Invalid parallel dimensions: product={total} does not match "
                f"world_size={self.world_size}"
            )

    # -- basic facts -------------------------------------------------------------------------
    def _sizes(self) -> tuple[int, ...]:
        return tuple(getattr(self, name) for name in _ORDER)

    @property
    def dp_world_size(self) -> int:
        return self.dp_replicate * self.dp_shard

    @property
    def dp_enabled(self) -> bool:
        return self.dp_world_size > 1

    @property
    def tp_enabled(self) -> bool:
        return self.tp > 1

    @property
    def pp_enabled(self) -> bool:
        return self.pp > 1

    @property
    def cp_enabled(self) -> bool:
        return self.cp > 1

    @property
    def ep_enabled(self) -> bool:
        return self.ep > 1

    @property
    def distributed_enabled(self) -> bool:
        return self.world_size > 1

    @property
    def global_rank(self) -> int:
        return int(os.environ.get("RANK", "0"))

    @property
    def local_rank(self) -> int:
        return int(os.environ.get("LOCAL_RANK", "0"))

    # -- coordinates -------------------------------------------------------------------------
    def _coordinates(self, rank: int) -> tuple[int, ...]:
        coords = []
        rest = int(rank)
        for size in reversed(self._sizes()):
            coords.append(rest % size)
            rest //= size
        return tuple(reversed(coords))

    def _rank_from_coordinates(self, coords: tuple[int, ...]) -> int:
        rank = 0
        for value, size in zip(coords, self._sizes(), strict=True):
            rank = rank * size + value
        return rank

    def coordinate(self, name: str, rank: int | None = None) -> int:
        rank = self.global_rank if rank is None else rank
        return self._coordinates(rank)[_ORDER.index(name)]

    def group_ranks(self, names: tuple[str, ...] | str, rank: int | None = None) -> list[int]:
        """Ranks that share every coordinate with ``rank`` except those in ``names``."""
        names = (names,) if isinstance(names, str) else tuple(names)
        rank = self.global_rank if rank is None else rank
        coords = list(self._coordinates(rank))
        axes = [_ORDER.index(name) for name in names]
        ranks = []
        for values in product(*(range(self._sizes()[axis]) for axis in axes)):
            for axis, value in zip(axes, values):
                coords[axis] = value
            ranks.append(self._rank_from_coordinates(tuple(coords)))
        return ranks

    def iter_groups(self, names: tuple[str, ...] | str) -> Iterable[list[int]]:
        """Every distinct group along ``names`` (each rank appears in exactly one)."""
        seen: set[int] = set()
        for rank in range(self.world_size):
            if rank in seen:
                continue
            ranks = self.group_ranks(names, rank)
            seen.update(ranks)
            yield ranks

    # -- named views used by the engine and by tests --------------------------------------------
    @property
    def pp_rank(self) -> int:
        return self.coordinate("pp")

    @property
    def dp_replicate_rank(self) -> int:
        return self.coordinate("dp_replicate")

    @property
    def dp_shard_rank(self) -> int:
        return self.coordinate("dp_shard")

    @property
    def cp_rank(self) -> int:
        return self.coordinate("cp")

    @property
    def tp_rank(self) -> int:
        return self.coordinate("tp")

    @property
    def ep_rank(self) -> int:
        return self.coordinate("ep")

    @property
    def dp_rank(self) -> int:
        return self.dp_replicate_rank * self.dp_shard + self.dp_shard_rank

    @property
    def is_first_pp_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_pp_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    def data_parallel_group_ranks(self, rank: int | None = None) -> list[int]:
        return self.group_ranks(("dp_replicate", "dp_shard"), rank)

    def tensor_parallel_group_ranks(self, rank: int | None = None) -> list[int]:
        return self.group_ranks("tp", rank)

    def context_parallel_group_ranks(self, rank: int | None = None) -> list[int]:
        return self.group_ranks("cp", rank)

    def expert_parallel_group_ranks(self, rank: int | None = None) -> list[int]:
        return self.group_ranks("ep", rank)

    def iter_all_data_parallel_groups(self) -> Iterable[list[int]]:
        return self.iter_groups(("dp_replicate", "dp_shard"))
