"""Mixture-of-experts kernels (router top-k, dispatch plan, permute / combine, quantile select)
against plain PyTorch references of the same ops."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from ohara_b200.ops._ext import ext

    return ext()


@pytest.mark.parametrize("gate_fn,normalize,bias", [("softmax", False, True), ("sigmoid", True, True),
                                                    ("sigmoid", False, False)])
@pytest.mark.parametrize("tokens,experts,k", [(1000, 64, 8), (257, 8, 2), (64, 256, 16)])
def test_route_matches_torch_topk(gate_fn, normalize, bias, tokens, experts, k):
    from ohara_b200.modules.routing import route_tokens
    from ohara_b200.ops.moe import route

    torch.manual_seed(0)
    logits = torch.randn(tokens, experts, device="cuda")
    router_bias = torch.randn(experts, device="cuda") * 0.3 if bias else torch.zeros(experts, device="cuda")
    want_alpha = bias
    indices, weights, alpha, counts = route(logits, router_bias if bias else None, k, gate_fn,
                                            normalize, want_alpha)
    ref_idx, ref_w, ref_alpha = route_tokens(logits, router_bias, k, gate_fn, want_alpha, normalize)
    assert torch.equal(indices.long(), ref_idx)
    assert torch.allclose(weights, ref_w, atol=1e-5, rtol=1e-5)
    if want_alpha:
        assert torch.allclose(alpha, ref_alpha.view(-1), atol=1e-6)
    assert torch.equal(counts.long(), torch.bincount(ref_idx.reshape(-1), minlength=experts))


def test_route_backward_matches_autograd():
    from ohara_b200.modules.routing import route_tokens
    from ohara_b200.ops.moe import route

    torch.manual_seed(1)
    for gate_fn, normalize in (("softmax", False), ("sigmoid", True), ("sigmoid", False)):
        base = torch.randn(300, 16, device="cuda")
        upstream = torch.randn(300, 4, device="cuda")
        a = base.clone().requires_grad_()
        route(a, None, 4, gate_fn, normalize, False)[1].mul(upstream).sum().backward()
        b = base.clone().requires_grad_()
        route_tokens(b, torch.zeros(16, device="cuda"), 4, gate_fn, False, normalize)[1].mul(upstream).sum().backward()
        assert torch.allclose(a.grad, b.grad, atol=1e-5, rtol=1e-4), gate_fn


def test_router_logits_keep_fp32_accuracy():
    from ohara_b200.ops.moe import router_logits

    torch.manual_seed(2)
    x = torch.randn(2048, 1024, device="cuda").bfloat16()
    w = (torch.randn(64, 1024, device="cuda") * 0.03).requires_grad_()
    exact = x.double() @ w.detach().double().t()
    got = router_logits(x, w)
    plain = x.float() @ w.detach().bfloat16().float().t()
    err = (got.double() - exact).abs().max().item()
    assert err < 2e-4 and err < 0.1 * (plain.double() - exact).abs().max().item()
    got.square().sum().backward()
    ref = (2 * exact.float()).t() @ x.float()
    assert (w.grad - ref).abs().max() / ref.abs().max() < 2e-2


def test_plan_permute_combine_round_trip(C):
    torch.manual_seed(3)
    tokens, k, experts, dim = 777, 4, 16, 64
    scores = torch.randn(tokens, experts, device="cuda")
    scores[:, 5] = -1e9  # an expert nobody picks
    indices = scores.topk(k, dim=-1).indices.int()
    counts = torch.bincount(indices.reshape(-1).long(), minlength=experts).int()
    dest_row, row_pair, tile_expert, k_offsets = C.moe_plan(indices, counts, 128)
    flat = indices.reshape(-1).long()
    rows = row_pair.numel()
    # every pair has its own row inside its expert's segment; segments are 128-aligned
    assert dest_row.unique().numel() == tokens * k
    assert torch.all((dest_row >= k_offsets[flat]) & (dest_row < k_offsets[flat + 1]))
    assert torch.all(k_offsets % 128 == 0) and int(k_offsets[-1]) <= rows
    assert torch.equal(k_offsets[1:] - k_offsets[:-1], (counts + 127) // 128 * 128)
    assert torch.equal(row_pair[dest_row.long()], torch.arange(tokens * k, device="cuda", dtype=torch.int32))
    assert int((row_pair >= 0).sum()) == tokens * k
    tile_of = torch.arange(rows // 128, device="cuda") * 128
    expected_tile = torch.searchsorted(k_offsets[1:].long().contiguous(), tile_of, right=True)
    expected_tile = torch.where(tile_of < k_offsets[-1], expected_tile, -1)
    assert torch.equal(tile_expert.long(), expected_tile)

    x = torch.randn(tokens, dim, device="cuda").bfloat16()
    x_pad = torch.full((rows, dim), 7.0, device="cuda", dtype=torch.bfloat16)
    C.moe_scatter_rows(x, dest_row, None, row_pair, x_pad, k)
    assert torch.equal(x_pad[dest_row.long()], x.repeat_interleave(k, dim=0))
    assert torch.all(x_pad[row_pair < 0] == 0)

    weights = torch.rand(tokens, k, device="cuda")
    other = torch.randn(tokens, dim, device="cuda").bfloat16()
    out, dot = C.moe_gather_combine(x_pad, dest_row, weights, other, k, True)
    picked = x_pad[dest_row.long()].float().view(tokens, k, dim)
    assert torch.allclose(out.float(), (picked * weights.unsqueeze(-1)).sum(1), atol=2e-2, rtol=2e-2)
    assert torch.allclose(dot, (picked * other.float().unsqueeze(1)).sum(-1), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("tokens,experts,rank", [(4096, 64, 512), (1000, 8, 1), (513, 16, 513)])
def test_quantile_select_is_exact(C, tokens, experts, rank):
    torch.manual_seed(4)
    logits = torch.randn(tokens, experts, device="cuda")
    alpha = torch.randn(tokens, device="cuda")
    total = torch.ones(experts, device="cuda")
    C.qb_quantile(logits, alpha, total, rank)
    expected = torch.topk((logits - alpha[:, None]).t(), rank, dim=-1).values[:, -1]
    assert torch.equal(total - 1, expected) or torch.allclose(total - 1, expected, atol=1e-6)


def test_grouped_moe_layer_matches_the_reference_loop_with_gradients():
    from ohara_b200.modules.moe_grouped import GroupedMoE

    torch.manual_seed(5)
    layer = GroupedMoE(256, 128, num_experts=16, num_experts_per_tok=4, num_shared_experts=1).cuda()
    with torch.no_grad():
        layer.w_down.normal_(std=0.05)
        layer.shared_down.weight.normal_(std=0.05)
    layer.train()
    # bf16-representable inputs: both paths then see the same router inputs and, up to the rare
    # near-tie, make the same routing decisions
    x = torch.randn(4, 300, 256, device="cuda").bfloat16().float()

    def run(fast: bool):
        layer.zero_grad()
        layer.expert_counts.zero_()
        layer.qb_beta_sum.zero_()
        layer.qb_beta_count.zero_()
        inp = x.clone().requires_grad_()
        if fast:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = layer(inp)
        else:
            flat = inp.reshape(-1, 256)
            indices, weights, logits, alpha = layer._route(flat)
            out = layer._dispatch_reference(flat, indices, weights) + layer._shared(flat)
            out = out.view_as(inp)
            layer._accumulate_qb(logits.detach(), alpha.detach())
            layer._record_load(indices)
        out.float().square().mean().backward()
        grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
        return out.detach().float(), inp.grad.clone(), grads, layer.expert_counts.clone(), layer.qb_beta_sum.clone()

    fast, slow = run(True), run(False)

    def close(a, b, tol, rows_allowed=0.0):
        """Relative error against the largest reference entry; `rows_allowed` is the fraction of
        rows that may be off (a token whose k-th and (k+1)-th experts swap places)."""
        a, b = a.float().reshape(-1, a.shape[-1]), b.float().reshape(-1, b.shape[-1])
        bad = ((a - b).abs().amax(dim=1) > tol * (b.abs().max().item() + 1e-6)).float().mean().item()
        return bad <= rows_allowed

    assert close(fast[0], slow[0], 3e-2, rows_allowed=0.01)
    assert close(fast[1], slow[1], 5e-2, rows_allowed=0.01)
    for name in slow[2]:
        assert close(fast[2][name].flatten(1) if fast[2][name].dim() > 1 else fast[2][name][None],
                     slow[2][name].flatten(1) if slow[2][name].dim() > 1 else slow[2][name][None],
                     8e-2, rows_allowed=0.02), name
    assert (fast[3] - slow[3]).abs().sum().item() <= 0.01 * slow[3].sum().item()
    assert torch.allclose(fast[4], slow[4], atol=5e-3)
