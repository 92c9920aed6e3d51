"""Serving kernels: fused RoPE + cache append, decode attention (bf16 and int8 caches), the fused
sampler, and the on-device decode loop of the chat engine, against PyTorch references."""

import math

import pytest
import torch

from helpers import chat_tokenizer, tiny_llama

pytestmark = pytest.mark.gpu


def _tables(dim, length):
    from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis

    cos, sin = precompute_freqs_cis(dim, length)
    return cos.cuda().float().contiguous(), sin.cuda().float().contiguous()


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 6, 128), (8, 2, 64), (16, 2, 128)])
def test_decode_step_matches_reference(int8, heads, kv_heads, dim):
    from ohara_b200.embeddings_pos.rotary import rope_reference
    from ohara_b200.modules.kv_cache import KVCache
    from ohara_b200.ops.attention import attention_reference
    from ohara_b200.ops.decode import decode_attention

    torch.manual_seed(0)
    batch, limit, prefix = 3, 700, 389
    cos, sin = _tables(dim, limit)
    fused = KVCache((batch, limit, kv_heads, dim), limit, device="cuda", dtype=torch.bfloat16, int8=int8)
    plain = KVCache((batch, limit, kv_heads, dim), limit, device="cuda", dtype=torch.bfloat16, int8=int8)
    keys = torch.randn(batch, prefix, kv_heads, dim, device="cuda").bfloat16()
    values = torch.randn(batch, prefix, kv_heads, dim, device="cuda").bfloat16()
    rotated = rope_reference(keys, cos[:prefix], sin[:prefix]).bfloat16()
    fused.forward(rotated, values, 0)
    plain.forward(rotated, values, 0)

    for step, position in enumerate((prefix, torch.tensor([prefix + 1], device="cuda", dtype=torch.int32))):
        q = torch.randn(batch, 1, heads, dim, device="cuda").bfloat16()
        k = torch.randn(batch, 1, kv_heads, dim, device="cuda").bfloat16()
        v = torch.randn(batch, 1, kv_heads, dim, device="cuda").bfloat16()
        at = prefix + step
        q_rot = fused.append_decode(q, k, v, cos, sin, position)
        out = decode_attention(q_rot, fused, position)

        ref_q = rope_reference(q, cos[at : at + 1], sin[at : at + 1]).bfloat16()
        ref_k = rope_reference(k, cos[at : at + 1], sin[at : at + 1]).bfloat16()
        all_k, all_v = plain.forward(ref_k, v, at)
        ref = attention_reference(ref_q, all_k, all_v, causal=True)
        assert torch.allclose(q_rot.float(), ref_q.float(), atol=2e-2)
        if int8:
            assert (fused.key[:, : at + 1].float() - plain.key[:, : at + 1].float()).abs().max() <= 2
        else:
            assert torch.equal(fused.key[:, : at + 1], plain.key[:, : at + 1])
            assert torch.equal(fused.value[:, : at + 1], plain.value[:, : at + 1])
        assert torch.allclose(out.float(), ref.float(), atol=3e-2 if int8 else 1e-2), (step, int8)


def test_decode_attention_split_counts_agree():
    from ohara_b200.ops._ext import ext

    torch.manual_seed(1)
    batch, length, heads, dim = 2, 1024, 4, 128
    q = torch.randn(batch, heads, dim, device="cuda").bfloat16()
    k = torch.randn(batch, length, heads, dim, device="cuda").bfloat16()
    v = torch.randn(batch, length, heads, dim, device="cuda").bfloat16()
    outs = [ext().decode_attention(q, k, v, [], 1000, None, 1 / math.sqrt(dim), splits)
            for splits in (1, 3, 16)]
    scores = torch.einsum("bhd,blhd->bhl", q.float(), k[:, :1000].float()) / math.sqrt(dim)
    ref = torch.einsum("bhl,blhd->bhd", scores.softmax(-1), v[:, :1000].float())
    for out in outs:
        assert torch.allclose(out.float(), ref, atol=1e-2)


def _reference_sample(logits, temperature, top_k, top_p, u, valid):
    """The sampler's definition in fp64: mask, top-k (ties kept), softmax, top-p (a token goes when
    the mass of strictly more likely tokens exceeds top_p), inverse CDF in index order."""
    x = logits.double()[:valid]
    if temperature == 0:
        return int(x.argmax())
    if 0 < top_k < x.numel():
        x = x.masked_fill(x < x.topk(top_k).values[-1], float("-inf"))
    p = torch.softmax(x / temperature, dim=-1)
    if 0 < top_p < 1:
        ordered, order = torch.sort(p, descending=True, stable=True)
        before = ordered.cumsum(0) - ordered
        keep = torch.zeros_like(p, dtype=torch.bool)
        keep[order[before <= top_p]] = True
        p = p * keep
    cdf = p.cumsum(0)
    target = min(max(u, 0.0), 0.99999994) * cdf[-1]
    return int(torch.searchsorted(cdf, target, right=True).clamp_max(x.numel() - 1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.0, 0, 1.0), (1.0, 0, 1.0), (0.8, 50, 0.9),
                                                     (1.3, 5, 1.0), (1.0, 0, 0.5)])
def test_sampler_follows_its_definition(dtype, temperature, top_k, top_p):
    from ohara_b200.ops.decode import sample

    torch.manual_seed(2)
    rows, vocab, valid = 24, 50304, 50257
    logits = (torch.randn(rows, vocab, device="cuda") * 3).to(dtype)
    uniforms = torch.rand(rows, device="cuda")
    tokens = sample(logits, temperature=temperature, top_k=top_k, top_p=top_p, valid_vocab=valid,
                    uniforms=uniforms)
    assert tokens.shape == (rows, 1) and int(tokens.max()) < valid
    agree = 0
    for row in range(rows):
        expected = _reference_sample(logits[row].cpu(), temperature, top_k, top_p,
                                     float(uniforms[row]), valid)
        agree += int(tokens[row, 0]) == expected
    # a draw that lands within float round-off of a CDF step may fall on the neighbouring token
    assert agree >= rows - 1


def test_sampler_draws_from_the_right_distribution():
    from ohara_b200.ops.decode import sample

    torch.manual_seed(3)
    probs = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    logits = probs.log().cuda().repeat(20000, 1)
    tokens = sample(logits, temperature=1.0, top_k=0, top_p=1.0)
    freq = torch.bincount(tokens.view(-1).cpu(), minlength=5).float() / 20000
    assert torch.allclose(freq, probs, atol=0.015)
    nucleus = sample(logits, temperature=1.0, top_k=0, top_p=0.7)
    assert set(nucleus.view(-1).tolist()) == {0, 1}, "0.5 + 0.25 exceeds 0.7 before the third token"
    top2 = sample(logits, temperature=1.0, top_k=2, top_p=1.0)
    freq2 = torch.bincount(top2.view(-1).cpu(), minlength=5).float() / 20000
    assert torch.allclose(freq2[:2], torch.tensor([2 / 3, 1 / 3]), atol=0.015) and freq2[2:].sum() == 0


def test_device_counters_advance_and_select_the_step():
    from ohara_b200.ops.decode import sample

    logits = torch.zeros(4, 1000, device="cuda")
    logits[:, 7] = 5.0
    out = torch.full((4, 3), -1, device="cuda", dtype=torch.int64)
    nxt = torch.zeros(4, device="cuda", dtype=torch.int64)
    counters = torch.tensor([0, 41, 0], device="cuda", dtype=torch.int32)
    for _ in range(3):
        sample(logits, temperature=0.0, out=out, next_input=nxt, counters=counters)
    assert torch.all(out == 7) and torch.all(nxt == 7)
    assert counters.tolist() == [3, 44, 0]


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_engine_device_loop_matches_the_eager_loop(kv_heads):
    from ohara_b200.chat_engine import ChatEngine, SamplingConfig

    tok = chat_tokenizer()
    model = tiny_llama(64, context=128, hidden_size=256, intermediate_size=512,
                       num_attention_heads=4, num_key_value_heads=kv_heads, seed=4)
    engine = ChatEngine(model, tok, device="cuda", dtype=torch.bfloat16)
    prompt = torch.randint(0, len(tok), (3, 17), device="cuda")
    greedy = SamplingConfig(temperature=0.0, max_new_tokens=24)

    graph = engine.generate_batch(prompt, greedy)
    eager_kernels = engine.generate_batch(prompt, greedy, cuda_graph=False)
    assert graph.shape == (3, 24) and torch.equal(graph, eager_kernels)
    assert int(graph.max()) < len(tok), "padding vocabulary rows are never produced"

    # The plain loop (host-side positions, full-forward prefill) must make the same choices except
    # where two logits are within bf16 round-off of each other.
    loop = engine.generate_batch(prompt, greedy, stop_on_end=True)
    width = min(loop.shape[1], 24)
    first_diff = (graph[:, :width] != loop[:, :width]).int().argmax(dim=1)
    same = (graph[:, :width] == loop[:, :width]).all(dim=1)
    assert bool(same.any()) or int(first_diff.min()) >= 4

    sampled = engine.generate_batch(prompt, SamplingConfig(temperature=1.0, top_k=50, top_p=0.9,
                                                           max_new_tokens=24), seed=11)
    again = engine.generate_batch(prompt, SamplingConfig(temperature=1.0, top_k=50, top_p=0.9,
                                                         max_new_tokens=24), seed=11)
    assert torch.equal(sampled, again) and int(sampled.max()) < len(tok)


def test_cached_decoding_matches_a_full_forward():
    model = tiny_llama(512, context=96, hidden_size=256, intermediate_size=512,
                       num_attention_heads=2, seed=5).cuda().bfloat16().eval()
    tokens = torch.randint(0, 512, (2, 40), device="cuda")
    with torch.inference_mode():
        full = model(tokens).float()
        for int8 in (False, True):
            cache = model.build_kv_cache(batch_size=2, int8=int8)
            pieces = [model(tokens[:, :32], cache, 0)]
            for position in range(32, 40):
                pieces.append(model(tokens[:, position : position + 1], cache, position))
            stepped = torch.cat(pieces, dim=1).float()
            tolerance = 0.25 if int8 else 0.08
            assert (stepped - full).abs().max() < tolerance * full.abs().max(), int8


@pytest.mark.parametrize("rows", [1, 3, 8, 13, 16])
@pytest.mark.parametrize("features,width", [(768, 768), (2048, 768), (768, 2048), (50304, 768), (100, 136)])
def test_skinny_gemm_matches_fp32(rows, features, width):
    from ohara_b200.ops import matmul_nt
    from ohara_b200.ops._ext import ext

    torch.manual_seed(rows)
    x = torch.randn(rows, width, device="cuda").bfloat16()
    w = torch.randn(features, width, device="cuda").bfloat16()
    out = torch.empty(rows, features, device="cuda", dtype=torch.bfloat16)
    assert ext().gemv(x, w, out), "decode-sized shapes must take the weight-streaming kernel"
    ref = x.float() @ w.float().t()
    assert (out.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    assert torch.equal(matmul_nt(x, w), out)
