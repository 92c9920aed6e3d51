"""Zig-zag context-parallel sharding: the host-side helpers and the decomposition of causal
attention into a local causal pass, a near pass and a far pass, checked on CPU with dense
attention (the GPU test runs the same decomposition on the flash kernels over two devices)."""

import math

import pytest
import torch

from ohara_b200.parallel.cp import (
    _merge,
    local_positions,
    shard_sequence,
    unshard_sequence,
    zigzag_blocks,
)


def dense_attention(q, k, v, causal):
    """``(B, T, H, D)`` operands -> output and log-sum-exp ``(B, H, T)``."""
    scores = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(q.shape[-1])
    if causal:
        mask = torch.ones(q.shape[1], k.shape[1], dtype=torch.bool).tril()
        scores = scores.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    out = torch.einsum("bhts,bshd->bthd", torch.softmax(scores, dim=-1), v)
    return out, lse


@pytest.mark.parametrize("world", [1, 2, 3, 4])
def test_shard_round_trip_and_positions(world):
    length = 2 * world * 5
    x = torch.arange(3 * length).view(3, length)
    shards = [shard_sequence(x, rank, world) for rank in range(world)]
    assert all(s.shape == (3, length // world) for s in shards)
    assert torch.equal(unshard_sequence(shards), x)
    for rank in range(world):
        pos = local_positions(rank, world, length // world)
        assert torch.equal(shards[rank][0], pos)
        early, late = zigzag_blocks(rank, world)
        assert early < late and early + late == 2 * world - 1
    with pytest.raises(ValueError):
        shard_sequence(torch.zeros(1, 2 * world + 1), 0, world)


@pytest.mark.parametrize("world", [2, 3, 4])
def test_three_passes_reproduce_causal_attention_with_equal_work(world):
    torch.manual_seed(world)
    h, heads, dim = 6, 2, 8
    length = 2 * world * h
    q, k, v = (torch.randn(2, length, heads, dim, dtype=torch.float64) for _ in range(3))
    reference, _ = dense_attention(q, k, v, causal=True)
    work = []
    for rank in range(world):
        ql, kl, vl = (shard_sequence(t, rank, world) for t in (q, k, v))
        out, lse = dense_attention(ql, kl, vl, causal=True)
        pairs = ql.shape[1] * (ql.shape[1] + 1) // 2
        if rank > 0:  # near: everyone's queries against the early halves of earlier ranks
            kn = torch.cat([shard_sequence(k, s, world)[:, :h] for s in range(rank)], dim=1)
            vn = torch.cat([shard_sequence(v, s, world)[:, :h] for s in range(rank)], dim=1)
            out_n, lse_n = dense_attention(ql, kn, vn, causal=False)
            out, lse = _merge(out, lse, out_n, lse_n)
            pairs += ql.shape[1] * kn.shape[1]
        if rank < world - 1:  # far: late-half queries against all tokens of later ranks
            kf = torch.cat([shard_sequence(k, s, world) for s in range(rank + 1, world)], dim=1)
            vf = torch.cat([shard_sequence(v, s, world) for s in range(rank + 1, world)], dim=1)
            out_f, lse_f = dense_attention(ql[:, h:], kf, vf, causal=False)
            late, _ = _merge(out[:, h:], lse[:, :, h:], out_f, lse_f)
            out = torch.cat((out[:, :h], late), dim=1)
            pairs += h * kf.shape[1]
        torch.testing.assert_close(out, shard_sequence(reference, rank, world), rtol=1e-5, atol=1e-5)  # the merge works in fp32
        work.append(pairs)
    assert max(work) - min(work) == 0, work  # every rank scores the same number of pairs


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_landing_layout_and_gradient_spans_are_consistent(world):
    from ohara_b200.parallel.cp import gradient_span, landing_layout

    count = 64
    for rank in range(world):
        near, far = landing_layout(rank, world, count)
        assert [src for src, _, _ in near] == list(range(rank))
        assert [src for src, _, _ in far] == list(range(rank + 1, world))
        cursor = 0
        for _, offset, elements in near + far:  # pieces tile the buffer without gaps or overlap
            assert offset == cursor
            cursor += elements
        assert cursor <= world * count  # fits the gather buffer of world * count elements
        assert all(elements == count // 2 for _, _, elements in near)
        assert all(elements == count for _, _, elements in far)
        # what this rank pulled from a source is what it later returns gradients for
        for src, _, elements in near + far:
            assert gradient_span(src, rank, count) == elements
