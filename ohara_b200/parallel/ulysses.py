"""Ulysses-style sequence parallelism for attention: all-to-all instead of a key/value exchange.

Every rank of the context-parallel group holds a shard of the sequence with all heads. Around
attention two all-to-alls re-partition the work: queries, keys and values go from
``(sequence shard, all heads)`` to ``(whole sequence, heads / world)``, ordinary causal flash
attention runs on the local heads, and the output goes back the same way. Compared with the
key/value exchange of :mod:`ohara_b200.parallel.cp` it moves ``q``, ``k``, ``v`` and the output
once each instead of ``k`` and ``v`` ``world - 1`` times, needs no merging of partial softmaxes,
and is limited to ``world <= heads``. The collective is the process group's ``all_to_all_single``
(NCCL on GPUs, gloo on CPUs), so this mode also runs on CPU ranks.

The sequence shards are the zig-zag shards of :func:`ohara_b200.parallel.cp.shard_sequence`, so
everything else about context parallelism (how a batch is cut, rotary positions, the loss scale,
the sharded optimizer over the group) is shared between the two modes; after the first all-to-all
the tokens are put into natural order with one gather so that the causal mask is the usual one.

The reference has neither mode (``cp`` is arithmetic in ohara/runtime/topology.py:33-38 and
nothing consumes it).
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import Tensor


class UlyssesWorkspace:
    """The group and the cached token orders of one context-parallel group."""

    def __init__(self, group) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._orders: dict[tuple[int, str], tuple[Tensor, Tensor]] = {}

    def orders(self, local_length: int, device) -> tuple[Tensor, Tensor]:
        """``(to_natural, to_gathered)`` index vectors for a gathered sequence of
        ``world * local_length`` tokens laid out rank after rank."""
        key = (local_length, str(device))
        cached = self._orders.get(key)
        if cached is None:
            from ohara_b200.parallel.cp import local_positions

            position = torch.cat([local_positions(r, self.world, local_length)
                                  for r in range(self.world)])
            to_natural = torch.argsort(position).to(device)
            to_gathered = position.to(device)
            cached = self._orders[key] = (to_natural, to_gathered)
        return cached


class _Exchange(torch.autograd.Function):
    """``(world, ...)`` blocks: block ``r`` goes to rank ``r``; the result holds the blocks
    received, indexed by source rank. Its own adjoint."""

    @staticmethod
    def forward(ctx, blocks: Tensor, group) -> Tensor:
        ctx.group = group
        blocks = blocks.contiguous()
        out = torch.empty_like(blocks)
        dist.all_to_all_single(out, blocks, group=group)
        return out

    @staticmethod
    def backward(ctx, grad: Tensor):
        grad = grad.contiguous()
        out = torch.empty_like(grad)
        dist.all_to_all_single(out, grad, group=ctx.group)
        return out, None


def sequence_to_heads(x: Tensor, workspace: UlyssesWorkspace) -> Tensor:
    """``(B, t, H, D)`` with all heads of this rank's tokens -> ``(B, world * t, H / world, D)``
    with this rank's heads of every token, rank after rank."""
    batch, steps, heads, dim = x.shape
    world = workspace.world
    blocks = x.reshape(batch, steps, world, heads // world, dim).permute(2, 0, 1, 3, 4)
    received = _Exchange.apply(blocks, workspace.group)            # (source, B, t, h, D)
    return received.permute(1, 0, 2, 3, 4).reshape(batch, world * steps, heads // world, dim)


def heads_to_sequence(x: Tensor, workspace: UlyssesWorkspace) -> Tensor:
    """Inverse of :func:`sequence_to_heads`: ``(B, world * t, h, D)`` -> ``(B, t, world * h, D)``."""
    batch, total, heads, dim = x.shape
    world = workspace.world
    steps = total // world
    blocks = x.reshape(batch, world, steps, heads, dim).permute(1, 0, 2, 3, 4)
    received = _Exchange.apply(blocks, workspace.group)            # (head group, B, t, h, D)
    return received.permute(1, 2, 0, 3, 4).reshape(batch, steps, world * heads, dim)


def ulysses_attention(q: Tensor, k: Tensor, v: Tensor, workspace: UlyssesWorkspace,
                      dropout_p: float = 0.0, training: bool = False) -> Tensor:
    """Causal attention over the whole sequence for rotated ``q (B, t, H, D)`` and
    ``k, v (B, t, Hk, D)`` of this rank's zig-zag shard; returns ``(B, t, H, D)``."""
    from ohara_b200 import ops

    world = workspace.world
    heads, kv_heads = q.shape[2], k.shape[2]
    if heads % world:
        raise ValueError(f"{heads} query heads do not divide over {world} ranks")
    if kv_heads % world:
        # grouped-query models with fewer key/value heads than ranks: repeat them just enough
        repeat = world // math.gcd(kv_heads, world)
        if heads % (kv_heads * repeat):
            raise ValueError(f"{kv_heads} key/value heads cannot be spread over {world} ranks")
        k = k.repeat_interleave(repeat, dim=2)
        v = v.repeat_interleave(repeat, dim=2)
    to_natural, to_gathered = workspace.orders(q.shape[1], q.device)
    whole = [sequence_to_heads(t, workspace).index_select(1, to_natural) for t in (q, k, v)]
    out = ops.attention(whole[0], whole[1], whole[2], causal=True, dropout_p=dropout_p,
                        training=training)
    return heads_to_sequence(out.index_select(1, to_gathered), workspace)
