"""Conway's Game of Life as a sequence-modelling task (reference: experiments/lifelm/life_ds.py:13-68,
whose dataset is unfinished: its iterator reads attributes that do not exist).

``next_state`` advances a whole batch of toroidal boards with one 3x3 convolution instead of the
reference's Python loop over cells. ``LifeDataset`` yields ``(board, next board)`` pairs along a
trajectory and starts a fresh random board when the trajectory dies out or enters a cycle (a board
it has produced before). ``boards_to_tokens`` lays a pair out as one token sequence
``current row-major | SEP | next row-major`` for a language model; the loss mask covers the second
half only."""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.utils.data import IterableDataset

DEAD, ALIVE, SEP = 0, 1, 2
VOCAB_SIZE = 3

_NEIGHBOURS = torch.ones(1, 1, 3, 3)
_NEIGHBOURS[0, 0, 1, 1] = 0.0


def next_state(boards: Tensor) -> Tensor:
    """One generation for ``(..., rows, cols)`` boards of 0/1 with wrap-around edges."""
    shape = boards.shape
    cells = boards.reshape(-1, 1, shape[-2], shape[-1]).float()
    padded = F.pad(cells, (1, 1, 1, 1), mode="circular")
    neighbours = F.conv2d(padded, _NEIGHBOURS.to(cells.device))
    alive = cells > 0.5
    survive = alive & ((neighbours == 2) | (neighbours == 3))
    born = ~alive & (neighbours == 3)
    return (survive | born).to(boards.dtype).reshape(shape)


def next_state_loops(board: Tensor) -> Tensor:
    """The same rule cell by cell (the oracle of ``next_state``'s test)."""
    rows, cols = board.shape
    out = torch.zeros_like(board)
    for i in range(rows):
        for j in range(cols):
            count = sum(int(board[(i + di) % rows, (j + dj) % cols])
                        for di in (-1, 0, 1) for dj in (-1, 0, 1) if (di, dj) != (0, 0))
            out[i, j] = int(count == 3 or (int(board[i, j]) == 1 and count == 2))
    return out


class LifeDataset(IterableDataset):
    def __init__(self, size: int, samples: int, density: float = 0.5, seed: int = 0) -> None:
        self.size, self.samples, self.density, self.seed = size, samples, density, seed

    def _fresh(self, generator: torch.Generator) -> Tensor:
        return (torch.rand(self.size, self.size, generator=generator) < self.density).long()

    def __iter__(self):
        generator = torch.Generator().manual_seed(self.seed)
        board = self._fresh(generator)
        seen = {board.numpy().tobytes()}
        for _ in range(self.samples):
            following = next_state(board)
            yield board, following
            key = following.numpy().tobytes()
            if key in seen or int(following.sum()) == 0:   # a cycle or an empty world: restart
                following = self._fresh(generator)
                seen = set()
                key = following.numpy().tobytes()
            seen.add(key)
            board = following


def boards_to_tokens(board: Tensor, following: Tensor) -> tuple[Tensor, Tensor]:
    """``(tokens, loss_mask)`` of length ``2 * cells + 1`` for one pair (or a batch of pairs)."""
    current = board.flatten(-2).long()
    target = following.flatten(-2).long()
    sep = torch.full_like(current[..., :1], SEP)
    tokens = torch.cat([current, sep, target], dim=-1)
    mask = torch.cat([torch.zeros_like(current), torch.zeros_like(sep), torch.ones_like(target)],
                     dim=-1).bool()
    return tokens, mask
