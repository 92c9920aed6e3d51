"""Every peer-memory kernel on ONE device: the ranks of a two- or three-way group are emulated one
after the other, each with its own buffers in the same GPU's memory and with the flags it would
wait for already set (kernels that wait on one another never run as concurrent launches on one
GPU). Covers the sharded optimizer's reduce-scatter / all-gather, the one-shot all-reduce, the
expert-parallel count exchange, plan, dispatch and combine, and the log-sum-exp merge of
context-parallel attention."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from ohara_b200.ops._ext import ext

    return ext()


@pytest.fixture(autouse=True)
def _status_clean(C):
    C.status(True)
    yield
    torch.cuda.synchronize()
    code, block, count, _ = C.status(True)
    assert code == 0, f"kernel wait timed out: code={code} block={block} count={count}"


def _pads(world, epoch):
    """One signal pad per emulated rank, every slot already at ``epoch``."""
    return [torch.full((1024,), epoch, dtype=torch.int32, device="cuda") for _ in range(world)]


@pytest.mark.parametrize("world,region", [(2, 4096), (3, 128 * 37)])
def test_reduce_scatter_mean_and_all_gather_kernels(C, world, region):
    torch.manual_seed(0)
    grads = [torch.randn(world * region, device="cuda").bfloat16() for _ in range(world)]
    pads = _pads(world, 1)
    mean = torch.stack([g.float() for g in grads]).mean(0)
    for rank in range(world):
        out = torch.full((region,), float("nan"), device="cuda")
        C.peer_reduce_scatter_mean([g.data_ptr() for g in grads], [p.data_ptr() for p in pads],
                                   out, region, rank, 1, 0.5)
        assert torch.allclose(out, mean[rank * region:(rank + 1) * region], atol=1e-6, rtol=1e-6)
    # all-gather: every rank holds only its own region, the kernel pulls the others
    full = torch.randn(world * region, device="cuda").bfloat16()
    weights = []
    for rank in range(world):
        mine = torch.zeros_like(full)
        mine[rank * region:(rank + 1) * region] = full[rank * region:(rank + 1) * region]
        weights.append(mine)
    pads = _pads(world, 2)
    for rank in range(world):
        C.peer_all_gather([w.data_ptr() for w in weights], [p.data_ptr() for p in pads],
                          region * 2, rank, 2, 0.5)
    for rank in range(world):
        assert torch.equal(weights[rank], full), rank


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_shot_all_reduce_kernel(C, dtype):
    world, n = 3, 5000
    torch.manual_seed(1)
    buffers = [torch.randn(n, device="cuda").to(dtype) for _ in range(world)]
    pads = _pads(world, 1)
    want = torch.stack([b.float() for b in buffers]).sum(0) * 0.5
    results = []
    for rank in range(world):
        out = torch.empty(n, device="cuda", dtype=dtype)
        C.peer_all_reduce([b.data_ptr() for b in buffers], [p.data_ptr() for p in pads], out, 0.5,
                          rank, 1, 0.5)
        results.append(out)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-6
    assert torch.allclose(results[0].float(), want, atol=tol, rtol=tol)
    assert all(torch.equal(results[0], other) for other in results[1:])  # bit-identical on all ranks


def test_expert_parallel_plan_dispatch_and_combine(C):
    """Two ranks, eight experts (four per rank), top-2: rows must land in the owner's buffer grouped
    by expert and padded to the tile height, and the combine must read them back weighted."""
    from ohara_b200.ops.moe import TILE

    world, experts, k, d, tokens = 2, 8, 2, 64, 300
    local = experts // world
    capacity = 8 * TILE
    torch.manual_seed(2)
    x = [torch.randn(tokens, d, device="cuda").bfloat16() for _ in range(world)]
    indices = [torch.stack([torch.randperm(experts, device="cuda")[:k] for _ in range(tokens)]).int()
               for _ in range(world)]
    weights = [torch.rand(tokens, k, device="cuda") for _ in range(world)]
    tables = [torch.zeros(world * experts, dtype=torch.int32, device="cuda") for _ in range(world)]
    for rank in range(world):
        counts = torch.bincount(indices[rank].reshape(-1).long(), minlength=experts).int()
        C.ep_publish_counts([t.data_ptr() for t in tables], counts, rank)
    assert torch.equal(tables[0], tables[1])  # every rank ends up with the same table
    plans = [C.ep_plan(tables[rank], indices[rank].contiguous(), rank, world, TILE, capacity)
             for rank in range(world)]
    from ohara_b200.utils.checks import validate_expert_parallel_plan

    for rank in range(world):  # the host-side validator agrees with what the kernels built
        validate_expert_parallel_plan(indices[rank], *plans[rank][:4], world=world,
                                      num_experts=experts, capacity_rows=capacity, tile=TILE)
    landing = [torch.full((capacity, d), float("nan"), device="cuda").bfloat16() for _ in range(world)]
    for rank in range(world):
        dest_rank, dest_row = plans[rank][0], plans[rank][1]
        assert int(dest_row.min()) >= 0  # nothing dropped at this capacity
        C.ep_push_rows(x[rank], dest_rank, dest_row, None, [b.data_ptr() for b in landing], k)
    torch.cuda.synchronize()
    for owner in range(world):
        k_offsets = plans[owner][3].tolist()
        tile_expert = plans[owner][2].tolist()
        assert all(offset % TILE == 0 for offset in k_offsets)
        for e in range(local):
            begin, end = k_offsets[e], k_offsets[e + 1]
            assert all(t == e for t in tile_expert[begin // TILE:end // TILE])
            want = torch.cat([x[r][(indices[r] == owner * local + e).any(1)] for r in range(world)])
            got = landing[owner][begin:begin + want.shape[0]]
            assert not torch.isnan(got.float()).any()
            # same multiset of rows (the order inside a segment is an implementation detail)
            assert torch.equal(torch.sort(got.float().sum(1)).values,
                               torch.sort(want.float().sum(1)).values)
    # "experts" double their input; the combine weights and sums the k outputs of every token
    outbox = [torch.nan_to_num(buf.float() * 2).bfloat16() for buf in landing]
    for rank in range(world):
        out, dots = C.ep_pull_combine([b.data_ptr() for b in outbox], plans[rank][0], plans[rank][1],
                                      weights[rank].reshape(-1).contiguous(), x[rank], k, d, True)
        want = 2 * x[rank].float() * weights[rank].sum(1, keepdim=True)
        assert (out.float() - want).abs().max() <= 2e-2 * want.abs().max()
        want_dots = 2 * x[rank].float().square().sum(1, keepdim=True).expand(-1, k)
        assert torch.allclose(dots, want_dots, rtol=2e-2, atol=1e-2)


def test_context_parallel_merge_of_two_key_sets_equals_attention_over_their_union(C):
    """The remote passes of context-parallel attention are merged into the local result through
    the log-sum-exp; merging attention over two disjoint key sets must equal attention over both."""
    from ohara_b200.ops.attention import attention_reference
    from ohara_b200.parallel.cp import _merge

    torch.manual_seed(3)
    b, t, h, hk, dim = 2, 256, 4, 2, 64
    q = torch.randn(b, t, h, dim, device="cuda").bfloat16()
    k = torch.randn(b, 2 * t, hk, dim, device="cuda").bfloat16()
    v = torch.randn(b, 2 * t, hk, dim, device="cuda").bfloat16()
    scale = dim ** -0.5
    out_a, lse_a = C.flash_attn_fwd(q, k[:, :t].contiguous(), v[:, :t].contiguous(), False, scale)
    out_b, lse_b = C.flash_attn_fwd(q, k[:, t:].contiguous(), v[:, t:].contiguous(), False, scale)
    merged, lse = _merge(out_a, lse_a, out_b, lse_b)
    want = attention_reference(q, k, v, causal=False, scale=scale)
    assert (merged.float() - want.float()).abs().max() <= 2e-2 * want.float().abs().max()
    whole, lse_whole = C.flash_attn_fwd(q, k, v, False, scale)
    assert torch.allclose(lse, lse_whole, atol=2e-2, rtol=1e-3)


def test_out_of_range_destination_is_reported_and_skipped(C):
    """A (rank, row) destination outside the peers' buffers must not be written to: the push
    records a bad-argument status, skips the pair and leaves every buffer untouched; the combine
    skips the read."""
    from ohara_b200 import ops

    d, capacity = 64, 256
    x = torch.ones(4, d, device="cuda").bfloat16()
    buffers = [torch.zeros(capacity, d, device="cuda").bfloat16() for _ in range(2)]
    dest_rank = torch.tensor([0, 1, 5, 1], dtype=torch.int32, device="cuda")    # rank 5 does not exist
    dest_row = torch.tensor([3, capacity, 7, 9], dtype=torch.int32, device="cuda")  # row == capacity
    C.ep_push_rows(x, dest_rank, dest_row, None, [b.data_ptr() for b in buffers], 1, capacity)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bad kernel argument"):
        ops.check_status()
    assert float(buffers[0][3].sum()) == d and float(buffers[1][9].sum()) == d   # the valid pairs
    assert float(buffers[0].sum()) == d and float(buffers[1].sum()) == d         # nothing else
    out, _ = C.ep_pull_combine([b.data_ptr() for b in buffers], dest_rank, dest_row, None, None, 1, d,
                               True, capacity)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bad kernel argument"):
        ops.check_status()
    assert out.float().sum(1).tolist() == [d, 0.0, 0.0, d]


@pytest.mark.parametrize("tokens,experts,k", [(700, 6, 2), (1, 5, 2), (4096, 64, 8)])
def test_dispatch_plan_tables_satisfy_the_host_side_validator(C, tokens, experts, k):
    """The tables of the single-GPU routing plan (and of a plan whose small capacity drops pairs
    under expert parallelism) pass the checks that ``OHARA_DEBUG_CHECKS=1`` switches on."""
    from ohara_b200.ops.moe import TILE, dispatch_plan
    from ohara_b200.utils.checks import validate_dispatch_plan, validate_expert_parallel_plan

    torch.manual_seed(3)
    indices = torch.stack([torch.randperm(experts, device="cuda")[:k] for _ in range(tokens)]).int()
    counts = torch.bincount(indices.reshape(-1).long(), minlength=experts).int()
    validate_dispatch_plan(indices, *dispatch_plan(indices, counts), TILE)
    if experts % 2 == 0:
        world, capacity = 2, 2 * TILE   # far too small for 4096 x 8 pairs: most are dropped
        tables = [torch.zeros(world * experts, dtype=torch.int32, device="cuda") for _ in range(world)]
        for rank in range(world):
            C.ep_publish_counts([t.data_ptr() for t in tables], counts, rank)
        for rank in range(world):
            plan = C.ep_plan(tables[rank], indices.contiguous(), rank, world, TILE, capacity)
            validate_expert_parallel_plan(indices, *plan[:4], world=world, num_experts=experts,
                                          capacity_rows=capacity, tile=TILE)
