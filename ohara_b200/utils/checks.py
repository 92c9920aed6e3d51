"""Host-side validation of the index tables that the routing kernels build on the device.

The permutation, grouped-GEMM and expert-parallel kernels index memory with values computed by
other kernels (destination rows, tile-to-expert tables, segment offsets). A wrong table does not
fail loudly: it corrupts a neighbouring row or reads a stale one. These checks read a table back to
the host and verify the invariants the consumers rely on; they synchronise, so they run only when
``OHARA_DEBUG_CHECKS=1`` is set (the mixture-of-experts layers call them then) or when a test calls
them directly. They take CPU tensors as well, which is how their own tests run.

The reference has no counterpart (its routing is index arithmetic in PyTorch, which raises on an
out-of-range index by itself: ohara/modules/moe_grouped.py:156-185).
"""

from __future__ import annotations

import os

import torch
from torch import Tensor


class PlanError(AssertionError):
    """An index table violates an invariant of the kernels that consume it."""


def debug_checks_enabled() -> bool:
    return os.environ.get("OHARA_DEBUG_CHECKS", "0") not in ("", "0", "false", "False")


def _fail(message: str) -> None:
    raise PlanError(message)


def validate_dispatch_plan(indices: Tensor, dest_row: Tensor, row_pair: Tensor, tile_expert: Tensor,
                           k_offsets: Tensor, tile: int) -> None:
    """Tables of ``ops.moe.dispatch_plan`` for int ``indices (N, k)``:

    * ``k_offsets (E+1,)`` is non-decreasing, starts at 0, every boundary a multiple of ``tile``
      and the last one within the buffer;
    * ``dest_row (N*k,)`` is a permutation into the buffer: in range, no row used twice, and the
      row of pair ``j`` lies in the segment of expert ``indices.flat[j]``;
    * ``row_pair (rows,)`` is the inverse: ``row_pair[dest_row[j]] == j`` and every other row is
      marked unused (negative);
    * ``tile_expert (rows / tile,)`` names, for every tile inside a segment, that segment's expert,
      and -1 for tiles past the last segment.
    """
    flat = indices.reshape(-1).long().cpu()
    dest = dest_row.long().cpu()
    pair = row_pair.long().cpu()
    tiles = tile_expert.long().cpu()
    offsets = k_offsets.long().cpu()
    rows = pair.numel()
    experts = offsets.numel() - 1
    if dest.numel() != flat.numel():
        _fail(f"dest_row has {dest.numel()} entries for {flat.numel()} pairs")
    if rows % tile or tiles.numel() != rows // tile:
        _fail(f"buffer of {rows} rows does not match {tiles.numel()} tiles of {tile}")
    if int(offsets[0]) != 0 or bool((offsets[1:] < offsets[:-1]).any()):
        _fail("k_offsets must start at 0 and never decrease")
    if bool((offsets % tile != 0).any()) or int(offsets[-1]) > rows:
        _fail("segment boundaries must be tile multiples inside the buffer")
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= experts):
        _fail("expert index out of range")
    if dest.numel():
        if int(dest.min()) < 0 or int(dest.max()) >= rows:
            _fail(f"destination row out of range [0, {rows})")
        if torch.unique(dest).numel() != dest.numel():
            _fail("two pairs share a destination row")
        begin, end = offsets[flat], offsets[flat + 1]
        wrong = (dest < begin) | (dest >= end)
        if bool(wrong.any()):
            j = int(wrong.nonzero()[0])
            _fail(f"pair {j} (expert {int(flat[j])}) placed at row {int(dest[j])} outside its "
                  f"segment [{int(begin[j])}, {int(end[j])})")
        if not torch.equal(pair[dest], torch.arange(dest.numel())):
            _fail("row_pair is not the inverse of dest_row")
    used = torch.zeros(rows, dtype=torch.bool)
    used[dest] = True
    if bool((pair[~used] >= 0).any()):
        _fail("a padding row is marked as holding a pair")
    counts = torch.bincount(flat, minlength=experts)
    if bool((offsets[1:] - offsets[:-1] < counts).any()):
        _fail("a segment is shorter than the number of pairs routed to its expert")
    tile_begin = torch.arange(tiles.numel()) * tile
    want = torch.searchsorted(offsets[1:].contiguous(), tile_begin, right=True)
    want = torch.where(tile_begin < offsets[-1], want, torch.full_like(want, -1))
    if not torch.equal(tiles, want):
        t = int((tiles != want).nonzero()[0])
        _fail(f"tile {t} is labelled expert {int(tiles[t])}, its rows belong to {int(want[t])}")


def validate_expert_parallel_plan(indices: Tensor, dest_rank: Tensor, dest_row: Tensor,
                                  tile_expert: Tensor, k_offsets: Tensor, *, world: int,
                                  num_experts: int, capacity_rows: int, tile: int) -> None:
    """Tables of ``EPWorkspace.plan`` as one rank sees them, for its own int ``indices (N, k)``:

    * ``dest_rank`` is the owner of each pair's expert (``expert // (num_experts / world)``);
    * ``dest_row`` is -1 (dropped) or a row below ``capacity_rows``; no two pairs of this rank
      share a ``(rank, row)`` slot;
    * this rank's ``k_offsets (local + 1,)`` never decreases, stays within ``capacity_rows`` and
      has tile-multiple boundaries except where the capacity clamps them;
    * ``tile_expert`` labels every tile below the last boundary with the local expert whose
      segment holds it and the rest with -1.
    """
    flat = indices.reshape(-1).long().cpu()
    rank_of = dest_rank.long().cpu()
    row_of = dest_row.long().cpu()
    tiles = tile_expert.long().cpu()
    offsets = k_offsets.long().cpu()
    if num_experts % world:
        _fail("experts do not divide over the ranks")
    local = num_experts // world
    if offsets.numel() != local + 1:
        _fail(f"k_offsets has {offsets.numel()} entries for {local} local experts")
    if rank_of.numel() != flat.numel() or row_of.numel() != flat.numel():
        _fail("one destination per pair expected")
    if flat.numel():
        if int(flat.min()) < 0 or int(flat.max()) >= num_experts:
            _fail("expert index out of range")
        if not torch.equal(rank_of, flat // local):
            _fail("dest_rank is not the owner of the pair's expert")
        if int(row_of.min()) < -1 or int(row_of.max()) >= capacity_rows:
            _fail(f"destination row outside [-1, {capacity_rows})")
        kept = row_of >= 0
        slots = rank_of[kept] * capacity_rows + row_of[kept]
        if torch.unique(slots).numel() != slots.numel():
            _fail("two pairs of this rank share a destination slot")
    if bool((offsets[1:] < offsets[:-1]).any()) or int(offsets[0]) < 0:
        _fail("k_offsets must never decrease")
    if int(offsets[-1]) > capacity_rows:
        _fail("a segment ends beyond the capacity")
    unclamped = offsets < capacity_rows
    if bool((offsets[unclamped] % tile != 0).any()):
        _fail("segment boundaries below the capacity must be tile multiples")
    if capacity_rows % tile or tiles.numel() < capacity_rows // tile:
        _fail("tile table shorter than the buffer")
    tile_begin = torch.arange(tiles.numel()) * tile
    want = torch.searchsorted(offsets[1:].contiguous(), tile_begin, right=True)
    want = torch.where(tile_begin < offsets[-1], want, torch.full_like(want, -1))
    if not torch.equal(tiles, want):
        t = int((tiles != want).nonzero()[0])
        _fail(f"tile {t} is labelled expert {int(tiles[t])}, its rows belong to {int(want[t])}")
