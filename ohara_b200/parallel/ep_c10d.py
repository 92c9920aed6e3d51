"""Expert parallelism over the process group's own all-to-all, for ranks without peer memory (CPU
ranks on gloo; any backend with ``all_to_all_single``).

The production path (:mod:`ohara_b200.parallel.ep`) moves rows with kernels that store into the
owners' buffers over NVLink and needs CUDA devices. This module gives the same layer semantics with
plain collectives, so that everything built around expert parallelism (how the engine shards the
experts, the two-part sharded optimizer, checkpoints with one optimizer state per expert-parallel
coordinate, the balancing statistics) runs and is tested on CPU ranks:

    sort this rank's (token, expert) pairs by expert  ->  exchange per-expert counts  ->
    all-to-all the rows to the experts' owners  ->  SwiGLU experts on the rows received  ->
    all-to-all the results back  ->  weight by the gates and sum per token

Dropless (no capacity limit at the receiver; a capacity factor on the layer still zeroes the
gates of the pairs it drops). Sizes are read on the host, so every step synchronises: this is a
functional path, not a fast one. The reference has no expert parallelism at all; the same
composition around its own modules is what ``baseline/compositions.py`` uses as the baseline arm.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor


class C10dEPWorkspace:
    """What :meth:`GroupedMoE.shard_experts` needs to know about the group."""

    uses_process_group = True  # the layer then exchanges rows with all-to-alls, not peer stores

    def __init__(self, group, num_experts: int) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("experts must divide over the ranks")
        self.num_experts = num_experts


class _Rows(torch.autograd.Function):
    """All-to-all of row blocks with per-rank row counts; the backward pass sends the gradients
    the opposite way."""

    @staticmethod
    def forward(ctx, rows: Tensor, send: list[int], receive: list[int], group) -> Tensor:
        ctx.send, ctx.receive, ctx.group = send, receive, group
        out = rows.new_empty(sum(receive), rows.shape[1])
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=receive,
                               input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, grad: Tensor):
        out = grad.new_empty(sum(ctx.send), grad.shape[1])
        dist.all_to_all_single(out, grad.contiguous(), output_split_sizes=ctx.send,
                               input_split_sizes=ctx.receive, group=ctx.group)
        return out, None, None, None


def expert_parallel_swiglu_c10d(flat_x: Tensor, indices: Tensor, weights: Tensor, w_gate: Tensor,
                                w_up: Tensor, w_down: Tensor, workspace: C10dEPWorkspace) -> Tensor:
    """``indices (N, k)``: global expert ids chosen for this rank's tokens; ``w_gate / w_up
    (E_local, d, h)`` and ``w_down (E_local, h, d)``: this rank's experts. Returns ``(N, d)``."""
    world, group = workspace.world, workspace.group
    local = workspace.num_experts // world
    tokens, k = indices.shape
    pair_expert = indices.reshape(-1).long()
    order = torch.argsort(pair_expert, stable=True)            # by expert, hence by owner rank
    pair_token = order // k
    per_expert = torch.bincount(pair_expert, minlength=workspace.num_experts)
    incoming = torch.empty_like(per_expert)                      # (source rank, my local expert)
    dist.all_to_all_single(incoming, per_expert, group=group)
    send = per_expert.view(world, local).sum(1).tolist()
    receive = incoming.view(world, local).sum(1).tolist()
    received = _Rows.apply(flat_x[pair_token], send, receive, group)
    # rows arrive source by source, inside a source expert by expert
    expert_of_row = torch.arange(local, device=flat_x.device).repeat(world).repeat_interleave(
        incoming.view(-1))
    result = torch.zeros_like(received)
    for expert in range(local):
        # (an expert without rows still goes through the products, with empty operands: its
        # weights then get a zero gradient instead of none, which data-parallel wrappers need)
        rows = (expert_of_row == expert).nonzero(as_tuple=True)[0]
        x = received[rows]
        gate, up, down = (w[expert].to(x.dtype) for w in (w_gate, w_up, w_down))
        result = result.index_add(0, rows, (F.silu(x @ gate) * (x @ up)) @ down)
    returned = _Rows.apply(result, receive, send, group)        # back in this rank's sorted order
    gates = weights.reshape(-1)[order].to(returned.dtype)
    return torch.zeros_like(flat_x).index_add(0, pair_token, returned * gates[:, None])
