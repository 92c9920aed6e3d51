"""ALiBi linear attention biases (https://arxiv.org/abs/2108.12409).

Reference behaviour: ohara/embeddings_pos/alibi.py:4-28.
"""

from __future__ import annotations

import torch


def get_alibi_mask(number_of_heads: int, max_seq_len: int) -> torch.Tensor:
    """Per-head distance penalties ``(heads, T, T)``; add to a causal mask before softmax.

    Entry ``[h, i, j]`` is ``-max(i + 1 - j, 0) * slope_h`` with ``slope_h = 2^(-(h+1) / (heads/8))``.
    """
    rows = torch.arange(1, max_seq_len + 1).view(1, -1, 1)
    cols = torch.arange(max_seq_len).view(1, 1, -1)
    distance = (rows - cols).clamp_min(0)
    slopes = 1 / 2 ** (torch.arange(1, number_of_heads + 1) / (number_of_heads / 8))
    return -distance.expand(number_of_heads, -1, -1) * slopes.view(number_of_heads, 1, 1)
