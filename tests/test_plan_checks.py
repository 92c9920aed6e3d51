"""Host-side validators of the routing tables: tables built the way the device kernels build them
(restated in PyTorch from the kernels' contracts) pass; every kind of corruption is named."""

import pytest
import torch

from ohara_b200.ops.grouped import TILE, build_dispatch_plan
from ohara_b200.utils.checks import (PlanError, validate_dispatch_plan,
                                     validate_expert_parallel_plan)


def _device_style_plan(indices, experts):
    """``ops.moe.dispatch_plan``'s outputs from the sort-based CPU plan: destination per pair in
    pair order, inverse table with -1 on padding rows."""
    _, sorted_dest, order, tile_expert, k_offsets, rows = build_dispatch_plan(indices, experts)
    dest_row = torch.empty_like(sorted_dest)
    dest_row[order] = sorted_dest
    row_pair = torch.full((rows,), -1, dtype=torch.int64)
    row_pair[dest_row] = torch.arange(dest_row.numel())
    return dest_row.int(), row_pair.int(), tile_expert, k_offsets


@pytest.fixture
def plan():
    torch.manual_seed(0)
    indices = torch.stack([torch.randperm(6)[:2] for _ in range(700)]).int()
    return (indices, *_device_style_plan(indices, 6))


def test_a_correct_plan_passes(plan):
    validate_dispatch_plan(*plan, TILE)
    # an expert without tokens and a single token are fine too
    lonely = torch.tensor([[0, 3]], dtype=torch.int32)
    validate_dispatch_plan(lonely, *_device_style_plan(lonely, 5), TILE)


@pytest.mark.parametrize("damage,message", [
    (lambda i, d, r, t, k: d.__setitem__(5, d[6]), "share a destination"),
    (lambda i, d, r, t, k: d.__setitem__(0, r.numel()), "out of range"),
    # pair 0 moved to a free padding row at the end of another expert's segment
    (lambda i, d, r, t, k: d.__setitem__(0, int(k[(int(i.reshape(-1)[0]) + 1) % 6 + 1]) - 1),
     "outside its segment"),
    (lambda i, d, r, t, k: r.__setitem__(int(d[3]), 9), "inverse"),
    (lambda i, d, r, t, k: t.__setitem__(0, 4), "tile 0 is labelled"),
    (lambda i, d, r, t, k: k.__setitem__(2, int(k[2]) + 8), "tile multiples"),
    (lambda i, d, r, t, k: k.__setitem__(0, TILE), "start at 0"),
])
def test_corrupted_tables_are_reported(plan, damage, message):
    indices, dest_row, row_pair, tile_expert, k_offsets = (t.clone() for t in plan)
    damage(indices, dest_row, row_pair, tile_expert, k_offsets)
    with pytest.raises(PlanError, match=message):
        validate_dispatch_plan(indices, dest_row, row_pair, tile_expert, k_offsets, TILE)


def _expert_parallel_tables(indices_by_rank, experts, capacity_rows):
    """What every rank's plan kernel computes from the published counts: for each owner the
    experts' tile-padded segments in order, inside them the source ranks in order; rows at or
    beyond the capacity are dropped and the owner's boundaries are clamped to it."""
    world = len(indices_by_rank)
    local = experts // world
    counts = torch.stack([torch.bincount(i.reshape(-1).long(), minlength=experts)
                          for i in indices_by_rank])                       # (source, expert)
    plans = []
    for rank, indices in enumerate(indices_by_rank):
        base = torch.zeros(experts, dtype=torch.int64)
        offsets = [0] * (local + 1)
        for owner in range(world):
            at = 0
            for el in range(local):
                e = owner * local + el
                base[e] = at + int(counts[:rank, e].sum())
                if owner == rank:
                    offsets[el] = min(at, capacity_rows)
                at += (int(counts[:, e].sum()) + TILE - 1) // TILE * TILE
            if owner == rank:
                offsets[local] = min(at, capacity_rows)
        flat = indices.reshape(-1).long()
        cursor = torch.zeros(experts, dtype=torch.int64)
        rows = torch.empty_like(flat)
        for j, e in enumerate(flat.tolist()):
            rows[j] = base[e] + cursor[e]
            cursor[e] += 1
        rows = torch.where(rows < capacity_rows, rows, torch.full_like(rows, -1))
        offsets = torch.tensor(offsets)
        tile_begin = torch.arange(capacity_rows // TILE) * TILE
        tiles = torch.searchsorted(offsets[1:].contiguous(), tile_begin, right=True)
        tiles = torch.where(tile_begin < offsets[-1], tiles, torch.full_like(tiles, -1))
        plans.append((indices, (flat // local).int(), rows.int(), tiles.int(), offsets.int()))
    return plans


@pytest.mark.parametrize("capacity_rows", [16 * TILE, 3 * TILE])
def test_expert_parallel_tables_pass_with_and_without_drops(capacity_rows):
    torch.manual_seed(1)
    per_rank = [torch.stack([torch.randperm(8)[:2] for _ in range(300)]).int() for _ in range(2)]
    for tables in _expert_parallel_tables(per_rank, 8, capacity_rows):
        validate_expert_parallel_plan(*tables, world=2, num_experts=8,
                                      capacity_rows=capacity_rows, tile=TILE)
    if capacity_rows == 3 * TILE:   # the small buffer really drops pairs
        assert any(bool((t[2] < 0).any()) for t in _expert_parallel_tables(per_rank, 8, capacity_rows))


@pytest.mark.parametrize("damage,message", [
    (lambda r, d, t, k: r.__setitem__(0, 1 - int(r[0])), "owner"),
    (lambda r, d, t, k: d.__setitem__(0, 16 * TILE), "outside"),
    (lambda r, d, t, k: d.__setitem__(1, int(d[[i for i in range(d.numel()) if r[i] == r[1] and i != 1][0]])),
     "share a destination slot"),
    (lambda r, d, t, k: k.__setitem__(1, int(k[2]) + TILE), "never decrease"),
    (lambda r, d, t, k: t.__setitem__(0, 3), "tile 0 is labelled"),
])
def test_corrupted_expert_parallel_tables_are_reported(damage, message):
    torch.manual_seed(1)
    per_rank = [torch.stack([torch.randperm(8)[:2] for _ in range(300)]).int() for _ in range(2)]
    indices, dest_rank, dest_row, tiles, offsets = (
        t.clone() for t in _expert_parallel_tables(per_rank, 8, 16 * TILE)[1])
    damage(dest_rank, dest_row, tiles, offsets)
    with pytest.raises(PlanError, match=message):
        validate_expert_parallel_plan(indices, dest_rank, dest_row, tiles, offsets, world=2,
                                      num_experts=8, capacity_rows=16 * TILE, tile=TILE)
