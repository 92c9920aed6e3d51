"""CORE evaluation on toy tasks with a model whose answers are known in advance
(reference suite: tests/test_core_eval.py:56-95)."""

from __future__ import annotations

import json

import pytest
import torch

from helpers import WordTokenizer
from ohara_b200.core_eval import (
    batch_sequences_lm,
    evaluate_core_from_bundle,
    evaluate_task,
    find_common_length,
    render_prompts_mc,
    render_prompts_schema,
)


class Parrot(torch.nn.Module):
    """Predicts that the next token is ``successor[token]`` with near certainty."""

    def __init__(self, vocab: int, successor: dict[int, int], max_seq_len: int | None = None):
        super().__init__()
        self.table = torch.full((vocab, vocab), -10.0)
        for current, following in successor.items():
            self.table[current, following] = 10.0
        if max_seq_len is not None:
            self.max_seq_len = max_seq_len

    def forward(self, ids):
        return self.table[ids]


@pytest.fixture()
def tok():
    return WordTokenizer()


def chain(tok, text: str) -> dict[int, int]:
    ids = tok.encode(text)
    return dict(zip(ids, ids[1:]))


def test_helpers(tok):
    assert find_common_length([[1, 2, 3], [1, 2, 4]]) == 2
    assert find_common_length([[9, 2, 3], [1, 2, 3]], "right") == 2
    with pytest.raises(ValueError):
        find_common_length([[1]], "up")
    item = {"query": "q", "choices": ["a", "b"], "gold": 1}
    assert render_prompts_mc(item, ": ", [item]) == ["q: b\n\nq: a", "q: b\n\nq: b"]
    schema = {"context_options": ["x", "y"], "continuation": "z", "gold": 0}
    assert render_prompts_schema(schema, " ") == ["x z", "y z"]
    with pytest.raises(ValueError, match="empty in token space"):
        batch_sequences_lm(tok, ["abc", "abc"])


def test_multiple_choice_picks_the_likeliest_choice(tok):
    model = Parrot(len(tok), chain(tok, "q:abc"))
    data = [{"query": "q", "choices": ["abc", "cba"], "gold": 0},
            {"query": "q", "choices": ["cba", "abc"], "gold": 1},
            {"query": "q", "choices": ["cba", "abc"], "gold": 0}]
    meta = {"task_type": "multiple_choice", "num_fewshot": 0, "continuation_delimiter": ":"}
    assert evaluate_task(model, tok, data, "cpu", meta) == pytest.approx(2 / 3)
    meta["num_fewshot"] = 1
    assert 0.0 <= evaluate_task(model, tok, data, "cpu", meta) <= 1.0


def test_schema_scores_the_shared_continuation(tok):
    model = Parrot(len(tok), chain(tok, "ab xyz"))
    data = [{"context_options": ["ab", "ba"], "continuation": "xyz", "gold": 0},
            {"context_options": ["ba", "ab"], "continuation": "xyz", "gold": 0}]
    meta = {"task_type": "schema", "num_fewshot": 0, "continuation_delimiter": " "}
    assert evaluate_task(model, tok, data, "cpu", meta) == pytest.approx(0.5)


def test_language_modeling_needs_every_token_right_and_respects_the_window(tok):
    # the rendered context is stripped, so the delimiter's trailing space never reaches the model
    model = Parrot(len(tok), chain(tok, "abcde"))
    data = [{"context": "ab", "continuation": "cde"}, {"context": "ab", "continuation": "ced"}]
    meta = {"task_type": "language_modeling", "num_fewshot": 0, "continuation_delimiter": " "}
    assert evaluate_task(model, tok, data, "cpu", meta) == pytest.approx(0.5)
    cropped = Parrot(len(tok), chain(tok, "abcde"), max_seq_len=3)
    assert evaluate_task(cropped, tok, data, "cpu", meta) == 0.0, "answer span cropped away"
    with pytest.raises(ValueError, match="Unsupported task type"):
        evaluate_task(model, tok, data, "cpu", {**meta, "task_type": "cloze"})


def test_bundle_centres_accuracy_on_the_random_baseline(tmp_path, tok):
    (tmp_path / "eval_data").mkdir()
    (tmp_path / "core.yaml").write_text(
        "icl_tasks:\n"
        "  - label: toy_mc\n    icl_task_type: multiple_choice\n    dataset_uri: mc.jsonl\n"
        "    num_fewshot: [0]\n    continuation_delimiter: ':'\n"
        "  - label: toy_lm\n    icl_task_type: language_modeling\n    dataset_uri: lm.jsonl\n"
        "    num_fewshot: [0]\n")
    (tmp_path / "eval_meta_data.csv").write_text("Eval Task,Random baseline\ntoy_mc,50\ntoy_lm,0\n")
    rows = [{"query": "q", "choices": ["abc", "cba"], "gold": 0}] * 3 + \
           [{"query": "q", "choices": ["abc", "cba"], "gold": 1}]
    (tmp_path / "eval_data" / "mc.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    (tmp_path / "eval_data" / "lm.jsonl").write_text(
        json.dumps({"context": "q:", "continuation": "abc"}) + "\n")
    model = Parrot(len(tok), chain(tok, "q:abc") | chain(tok, "q: abc"))
    out = evaluate_core_from_bundle(model, tok, "cpu", tmp_path)
    assert out["results"]["toy_mc"] == pytest.approx(0.75)
    assert out["centered_results"]["toy_mc"] == pytest.approx(0.5)
    assert out["core_metric"] == pytest.approx((0.5 + out["centered_results"]["toy_lm"]) / 2)
    limited = evaluate_core_from_bundle(model, tok, "cpu", tmp_path, max_per_task=1)
    assert limited["results"]["toy_mc"] in (0.0, 1.0)
