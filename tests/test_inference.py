"""Plain text generation helper (reference suite: tests/test_inference.py:45-81)."""

from __future__ import annotations

import pytest
import torch

from helpers import WordTokenizer, tiny_llama
from ohara_b200.inference import Inference


class Spy(torch.nn.Module):
    """Wraps a model and records the shape of every input and the position it was called at."""

    def __init__(self, model):
        super().__init__()
        self.model, self.config, self.calls = model, model.config, []

    def build_kv_cache(self, batch_size: int = 1):
        return self.model.build_kv_cache(batch_size)

    def forward(self, ids, kv_cache=None, position=None):
        self.calls.append((tuple(ids.shape), position))
        return self.model(ids, kv_cache, position) if kv_cache is not None else self.model(ids)


@pytest.fixture()
def tok():
    return WordTokenizer()


def test_sampler_is_greedy_at_zero_temperature_and_defaults():
    logits = torch.tensor([[[0.0, 3.0, 1.0]]])
    assert Inference.sampler(logits, temperature=0).tolist() == [[1]]
    assert Inference.sampler(logits).tolist() == [[1]]
    assert Inference.sampler(logits, temperature=1.0, top_p=1e-3).tolist() == [[1]]


def test_cached_and_uncached_generation_agree(tok):
    model = tiny_llama(len(tok))
    cached, plain = Spy(model), Spy(model)
    text = Inference(cached, tok, "cpu").generate("abc", temperature=0, max_new_tokens=5, stream=False)
    same = Inference(plain, tok, "cpu", use_kv_cache=False).generate(
        "abc", temperature=0, max_new_tokens=5, stream=False)
    assert text == same and text.startswith("abc") and len(text) > len("abc")
    produced = len(tok.encode(text)) - 3
    # prefill with the whole prompt, then one token per step at increasing positions
    assert cached.calls[0] == ((1, 3), 0)
    assert cached.calls[1 : 1 + produced] == [((1, 1), 3 + i) for i in range(produced)][: len(cached.calls) - 1]
    assert [shape for shape, _ in plain.calls[:3]] == [(1, 3), (1, 4), (1, 5)]


def test_generation_guards(tok):
    engine = Inference(tiny_llama(len(tok), context=8), tok, "cpu")
    with pytest.raises(ValueError, match="at least one token"):
        engine.generate("", stream=False)
    with pytest.raises(ValueError, match="negative"):
        engine.generate("ab", max_new_tokens=-1, stream=False)
    with pytest.raises(ValueError, match="exceeds"):
        engine.generate("a" * 9, stream=False)
    assert len(tok.encode(engine.generate("abcdef", temperature=0, max_new_tokens=50, stream=False))) <= 8
