"""Chat format, finetuning data, sampling, the chat engine and the web UI.

Behaviour checked here follows the reference suite (tests/test_chat.py:87-561).
"""

from __future__ import annotations

import json
import threading
import urllib.error
import urllib.request

import pytest
import torch

from helpers import WordTokenizer, chat_tokenizer, exchange, tiny_llama
from ohara_b200.chat import (
    ASSISTANT_END,
    ASSISTANT_START,
    CHAT_SPECIAL_TOKENS,
    OUTPUT_START,
    PYTHON_START,
    USER_END,
    USER_START,
    add_chat_tokens,
    normalize_messages,
    render_conversation,
    render_for_completion,
    resize_token_embeddings,
    special_token_ids,
    training_pair,
)
from ohara_b200.chat_engine import ChatEngine, SamplingConfig, config_from_state_dict, sample_next_token
from ohara_b200.sft import BestFitPacker, ConversationDataset, gsm8k_answer_parts, render_multiple_choice
from ohara_b200.webui.server import create_server


@pytest.fixture()
def tok():
    return chat_tokenizer()


# -- rendering -------------------------------------------------------------------------------------
def test_adding_chat_tokens_twice_grows_the_vocabulary_once():
    tokenizer = WordTokenizer()
    base = len(tokenizer)
    assert add_chat_tokens(tokenizer) == len(CHAT_SPECIAL_TOKENS)
    assert add_chat_tokens(tokenizer) == 0
    assert len(tokenizer) == base + len(CHAT_SPECIAL_TOKENS)


def test_special_ids_need_the_chat_tokens():
    with pytest.raises(ValueError, match="missing chat special tokens"):
        special_token_ids(WordTokenizer())


def test_only_the_assistant_side_is_supervised(tok):
    ids, mask = render_conversation(tok, exchange("hi", "yo")["messages"])
    special = special_token_ids(tok)
    assert ids[0] == tok.bos_token_id and mask[0] == 0
    assert ids[1] == special[USER_START] and ids[4] == special[USER_END]
    assert ids[5] == special[ASSISTANT_START] and mask[5] == 0
    supervised = [i for i, keep in zip(ids, mask) if keep]
    assert supervised == tok.encode("yo") + [special[ASSISTANT_END]]


def test_system_prompt_joins_the_first_user_turn(tok):
    messages = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"},
                {"role": "assistant", "content": "ok"}]
    turns = normalize_messages(messages)
    assert [t["role"] for t in turns] == ["user", "assistant"]
    assert turns[0]["content"] == "be brief\n\nhi"
    assert messages[1]["content"] == "hi", "the caller's list must not be edited"


@pytest.mark.parametrize("roles", [("assistant", "user"), ("user", "user"), ("system", "assistant")])
def test_out_of_order_roles_are_refused(roles):
    with pytest.raises(ValueError):
        normalize_messages([{"role": r, "content": "x"} for r in roles])


def test_tool_calls_are_supervised_but_tool_output_is_not(tok):
    answer = [{"type": "text", "text": "a"}, {"type": "python", "text": "1+1"},
              {"type": "python_output", "text": "2"}, {"type": "text", "text": "b"}]
    ids, mask = render_conversation(tok, exchange("q", answer)["messages"])
    special = special_token_ids(tok)
    at = {name: ids.index(special[name]) for name in (PYTHON_START, OUTPUT_START)}
    assert mask[at[PYTHON_START]] == 1 and mask[at[PYTHON_START] + 1] == 1
    assert mask[at[OUTPUT_START]] == 0 and mask[at[OUTPUT_START] + 1] == 0
    assert mask[-1] == 1 and ids[-1] == special[ASSISTANT_END]
    with pytest.raises(ValueError, match="unknown assistant content part"):
        render_conversation(tok, exchange("q", [{"type": "image", "text": ""}])["messages"])


def test_rendering_truncates(tok):
    ids, mask = render_conversation(tok, exchange("q" * 50, "a" * 50)["messages"], max_tokens=20)
    assert len(ids) == len(mask) == 20


def test_training_pair_shifts_by_one(tok):
    ids, mask = render_conversation(tok, exchange("hi", "yo")["messages"])
    inputs, targets = training_pair(ids, mask)
    assert inputs == ids[:-1]
    assert targets == [t if m else -1 for t, m in zip(ids[1:], mask[1:])]
    with pytest.raises(ValueError):
        training_pair([1], [0])
    with pytest.raises(ValueError):
        training_pair([1, 2], [0])


def test_completion_prompt_ends_with_assistant_start(tok):
    start = special_token_ids(tok)[ASSISTANT_START]
    open_turn = render_for_completion(tok, [{"role": "user", "content": "hi"}])
    assert open_turn[-1] == start and open_turn.count(start) == 1
    with_reply = render_for_completion(tok, exchange("hi", "old")["messages"])
    assert with_reply == open_turn, "a trailing assistant message is dropped"
    with pytest.raises(ValueError):
        render_for_completion(tok, [{"role": "assistant", "content": "x"}])


# -- vocabulary growth ---------------------------------------------------------------------------
def test_resize_keeps_trained_rows_and_tying(tok):
    model = tiny_llama(40, weight_tying=True)
    before = model.token_emb.weight.detach().clone()
    resize_token_embeddings(model, 48)
    assert model.token_emb.weight.shape == (48, 32)
    assert torch.equal(model.token_emb.weight[:40], before)
    assert model.vocab_proj.weight is model.token_emb.weight
    assert model(torch.randint(0, 48, (2, 8))).shape == (2, 8, 48)


def test_resize_untied_same_size_and_shrink(tok):
    model = tiny_llama(40, weight_tying=False)
    head = model.vocab_proj.weight.detach().clone()
    assert resize_token_embeddings(model, 40) is model
    resize_token_embeddings(model, 44)
    assert torch.equal(model.vocab_proj.weight[:40], head)
    assert model.vocab_proj.weight is not model.token_emb.weight
    with pytest.raises(ValueError, match="shrink"):
        resize_token_embeddings(model, 30)


# -- finetuning data -------------------------------------------------------------------------------
def _conversations(count=40):
    return [exchange("q" * (i % 7 + 1), "a" * (i % 5 + 1)) for i in range(count)]


def _dataset(tok, rows=None, **options):
    settings = dict(max_length=64, buffer_size=8, infinite=False, seed=0)
    settings.update(options)
    return ConversationDataset(rows or _conversations(), tok, **settings)


def test_packed_rows_are_well_formed(tok):
    rows = list(_dataset(tok))
    assert rows
    for inputs, targets in rows:
        assert inputs.shape == targets.shape == (64,)
        assert inputs.dtype == targets.dtype == torch.long
        assert inputs[0].item() == tok.bos_token_id, "rows start at a conversation boundary"
        keep = targets != -1
        assert keep.any()
        assert torch.equal(targets[:-1][keep[:-1]], inputs[1:][keep[:-1]])


def test_every_conversation_is_packed_exactly_once(tok):
    end = special_token_ids(tok)[ASSISTANT_END]
    seen = sum(int((inputs == end).sum()) + int(targets[-1] == end) for inputs, targets in _dataset(tok))
    assert seen == 40


def test_infinite_mode_keeps_going_and_malformed_rows_are_dropped(tok):
    one_epoch = len(list(_dataset(tok)))
    stream = iter(_dataset(tok, infinite=True))
    assert len([next(stream) for _ in range(3 * one_epoch)]) == 3 * one_epoch
    rows = _conversations(6) + [{"messages": [{"role": "assistant", "content": "x"}]},
                                {"messages": [{"role": "user", "content": "only a question"}]}]
    end = special_token_ids(tok)[ASSISTANT_END]
    kept = sum(int((i == end).sum()) + int(t[-1] == end) for i, t in _dataset(tok, rows))
    assert kept == 6


def test_data_shards_split_the_conversations(tok):
    end = special_token_ids(tok)[ASSISTANT_END]
    counts = []
    for rank in range(2):
        data = _dataset(tok, data_rank=rank, data_world_size=2, shuffle=False)
        counts.append(sum(int((i == end).sum()) + int(t[-1] == end) for i, t in data))
    assert counts == [20, 20]
    with pytest.raises(ValueError):
        _dataset(tok, data_rank=0)
    with pytest.raises(ValueError):
        ConversationDataset([], tok, max_length=8)


def test_best_fit_prefers_the_largest_item_that_fits():
    items = [([1] * 6, [1] * 6), ([2] * 3, [1] * 3), ([3] * 4, [1] * 4)]
    rows = list(BestFitPacker(capacity=10, buffer_size=3, pad_token_id=0).rows(iter(items)))
    assert rows[0][0] == [1] * 6 + [3] * 4
    assert rows[1][0] == [2] * 3 + [0] * 7 and rows[1][1] == [1] * 3 + [0] * 7


def test_prompt_helpers():
    text = render_multiple_choice("capital?", ["paris", "rome"])
    assert "=A" in text and "=B" in text and text.rstrip().endswith("answer.")
    parts = gsm8k_answer_parts("add <<1+1=2>>2 apples\n#### 2")
    kinds = [p["type"] for p in parts]
    assert kinds.count("python") == 1 and kinds.count("python_output") == 1
    assert parts[kinds.index("python")]["text"] == "1+1"


# -- sampling ----------------------------------------------------------------------------------------
def test_sampling_rules():
    logits = torch.tensor([[[0.1, 2.0, 0.3, 1.5]]])
    assert sample_next_token(logits, SamplingConfig(temperature=0.0)).tolist() == [[1]]
    draws = {int(sample_next_token(logits, SamplingConfig(temperature=5.0, top_k=2, top_p=1.0)))
             for _ in range(200)}
    assert draws <= {1, 3} and len(draws) == 2
    nucleus = {int(sample_next_token(logits, SamplingConfig(temperature=1.0, top_p=0.01)))
               for _ in range(50)}
    assert nucleus == {1}, "the most likely token always survives top-p"
    config = SamplingConfig(temperature=1.0)
    first = [int(sample_next_token(logits, config, torch.Generator().manual_seed(7))) for _ in range(1)]
    again = [int(sample_next_token(logits, config, torch.Generator().manual_seed(7))) for _ in range(1)]
    assert first == again
    for bad in (dict(temperature=-1), dict(top_p=1.5), dict(top_k=-1), dict(max_new_tokens=0)):
        with pytest.raises(ValueError):
            SamplingConfig(**bad)


# -- chat engine -------------------------------------------------------------------------------------
def _engine(tok, forced=None, context=64):
    model = tiny_llama(len(tok), context=context)
    if forced is not None:  # make the head emit one token whatever the input
        with torch.no_grad():
            model.vocab_proj.weight.zero_()
            model.vocab_proj.weight[forced] = 5.0
            model.token_emb.weight.fill_(1.0)
    return ChatEngine(model, tok, device="cpu", dtype=torch.float32)


def test_config_is_recovered_from_a_state_dict(tok):
    model = tiny_llama(len(tok), context=128, num_key_value_heads=1, weight_tying=False)
    rebuilt = config_from_state_dict(model.state_dict())
    for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                 "num_attention_heads", "num_key_value_heads", "max_sequence_length", "weight_tying"):
        assert getattr(rebuilt, name) == getattr(model.config, name), name


def test_generation_stops_at_the_end_token_or_the_budget(tok):
    hello = [{"role": "user", "content": "hi"}]
    end = special_token_ids(tok)[ASSISTANT_END]
    assert _engine(tok, forced=end).generate(hello, SamplingConfig(temperature=0.0)) == ""
    letter = tok.get_vocab()["h"]
    text = _engine(tok, forced=letter).generate(hello, SamplingConfig(temperature=0.0, max_new_tokens=5))
    assert text == "hhhhh"


def test_stream_batch_and_history_handling(tok):
    engine = _engine(tok)
    hello = [{"role": "user", "content": "hi"}]
    greedy = SamplingConfig(temperature=0.0, max_new_tokens=6)
    assert "".join(engine.generate_stream(hello, greedy)) == engine.generate(hello, greedy)
    prompt = torch.tensor([engine.render_prompt(hello)] * 2)
    rows = engine.generate_batch(prompt, greedy)
    assert rows.shape == (2, 6) and torch.equal(rows[0], rows[1])
    history = []
    for turn in range(12):
        history += exchange(f"question {turn}", f"answer {turn}")["messages"]
    history.append({"role": "user", "content": "latest"})
    ids = engine.render_prompt(history)
    assert len(ids) < 64 and tok.decode(ids).endswith("latest" + USER_END + ASSISTANT_START)
    with pytest.raises(ValueError):
        engine.render_prompt([{"role": "user", "content": "x" * 500}])
    info = engine.metadata()
    assert info["context_length"] == 64 and info["vocab_size"] == len(tok) and info["parameters"] > 0


# -- web UI ------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def server_url():
    tokenizer = chat_tokenizer()
    engine = _engine(tokenizer, forced=tokenizer.get_vocab()["h"])
    server = create_server(engine, host="127.0.0.1", port=0,
                           sampling=SamplingConfig(temperature=0.0, max_new_tokens=4))
    thread = threading.Thread(target=server.serve_forever, daemon=True)
    thread.start()
    yield f"http://127.0.0.1:{server.server_address[1]}"
    server.shutdown()
    server.server_close()
    thread.join(timeout=5)


def _get(url):
    with urllib.request.urlopen(url, timeout=10) as response:
        return response.status, response.read()


def _post(url, payload):
    request = urllib.request.Request(url, data=json.dumps(payload).encode(), method="POST",
                                     headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(request, timeout=30) as response:
        return response.status, response.read().decode()


def test_web_ui_pages_and_info(server_url):
    status, page = _get(server_url + "/")
    assert status == 200 and b"<html" in page.lower()
    for asset in ("/static/app.js", "/static/style.css"):
        assert _get(server_url + asset)[0] == 200
    info = json.loads(_get(server_url + "/api/info")[1])
    assert info["model"]["context_length"] == 64
    assert info["defaults"]["max_new_tokens"] == 4
    for missing in ("/nope", "/static/../server.py", "/static/%2e%2e/server.py"):
        with pytest.raises(urllib.error.HTTPError) as failure:
            _get(server_url + missing)
        assert failure.value.code in (403, 404)


def test_web_ui_chat_streams_and_validates(server_url):
    status, body = _post(server_url + "/api/chat", {"messages": [{"role": "user", "content": "hi"}]})
    assert status == 200
    events = [json.loads(line[len("data: "):]) for line in body.splitlines() if line.startswith("data: ")]
    assert "".join(e.get("delta", "") for e in events) == "hhhh"
    assert events[-1].get("done") is True
    for bad in ({}, {"messages": []}, {"messages": [{"role": "robot", "content": "x"}]},
                {"messages": [{"role": "user", "content": "x"}], "temperature": -2}):
        with pytest.raises(urllib.error.HTTPError) as failure:
            _post(server_url + "/api/chat", bad)
        assert failure.value.code == 400
