"""Token bins, tokenizer loading, streaming text datasets and corpus staging.

Behaviour checked here follows the reference suites (tests/test_tokenbin.py:43-203,
tests/test_tokenizer.py:47-117, tests/test_tokenizer_hookup.py:42-140,
tests/test_prepare_scaling_data.py:45-111).
"""

from __future__ import annotations

import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import WordTokenizer
from ohara_b200 import dataset as dataset_module
from ohara_b200 import tokenizer as tokenizer_module
from ohara_b200.dataset import StreamingTextDataset
from ohara_b200.tokenbin import (
    MAX_VOCAB,
    TokenBinDataset,
    read_token_bin_metadata,
    write_token_bin,
)
from ohara_b200.tokenizer import get_token_bytes, load_tokenizer

EXAMPLES = Path(__file__).resolve().parents[1] / "examples"
DOCS = ["the quick brown fox", "jumps over", "the lazy dog again and again"] * 20


def load_example(name: str):
    spec = importlib.util.spec_from_file_location(f"example_{name}", EXAMPLES / f"{name}.py")
    module = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = module
    spec.loader.exec_module(module)
    return module


@pytest.fixture()
def tok():
    return WordTokenizer()


@pytest.fixture()
def corpus_bin(tmp_path, tok):
    path = tmp_path / "train.bin"
    write_token_bin(DOCS, tok, path, log=False)
    return path


# -- writer ------------------------------------------------------------------------------------------
def test_bin_holds_boundary_separated_documents(tmp_path, tok):
    path = tmp_path / "x.bin"
    meta = write_token_bin(["ab", "", None, 7, "cd"], tok, path, batch_size=1, log=False)
    stored = np.fromfile(path, dtype=np.uint16).tolist()
    assert stored == [0] + tok.encode("ab") + [0] + tok.encode("cd")
    assert meta == read_token_bin_metadata(path)
    assert meta["tokens"] == 6 and meta["documents"] == 2 and meta["vocab_size"] == len(tok)
    assert meta["dtype"] == "uint16" and meta["boundary_token_id"] == 0
    assert len(list(tmp_path.iterdir())) == 2, "no temporary file is left behind"


def test_writer_refuses_empty_streams_and_wide_vocabularies(tmp_path, tok):
    with pytest.raises(RuntimeError, match="empty"):
        write_token_bin(["", None], tok, tmp_path / "e.bin", log=False)
    assert not (tmp_path / "e.bin").exists()
    tok.add_special_tokens({"additional_special_tokens": [f"<x{i}>" for i in range(MAX_VOCAB)]})
    with pytest.raises(ValueError, match="exceeds"):
        write_token_bin(["ab"], tok, tmp_path / "w.bin", log=False)


# -- reader ------------------------------------------------------------------------------------------
def test_blocks_are_shifted_views_of_the_file(corpus_bin):
    data = TokenBinDataset(corpus_bin, max_length=16, shuffle=False, infinite=False)
    stored = np.fromfile(corpus_bin, dtype=np.uint16).astype(np.int64)
    blocks = list(data)
    assert len(blocks) == data.num_blocks == len(stored) // 17
    for index, (inputs, targets) in enumerate(blocks):
        assert inputs.shape == targets.shape == (16,) and inputs.dtype == torch.long
        assert inputs.tolist() == stored[index * 17 : index * 17 + 16].tolist()
        assert targets.tolist() == stored[index * 17 + 1 : index * 17 + 17].tolist()


def test_shards_shuffle_epochs_and_resume(corpus_bin):
    def first_tokens(**options):
        settings = dict(max_length=16, shuffle=False, infinite=False)
        settings.update(options)
        return [tuple(x.tolist()) for x, _ in TokenBinDataset(corpus_bin, **settings)]

    everything = first_tokens()
    halves = [first_tokens(data_rank=r, data_world_size=2) for r in range(2)]
    assert sorted(halves[0] + halves[1]) == sorted(everything)
    assert len(halves[0]) - len(halves[1]) in (0, 1)
    shuffled = first_tokens(shuffle=True, seed=3)
    assert shuffled != everything and sorted(shuffled) == sorted(everything)
    assert first_tokens(shuffle=True, seed=3) == shuffled
    assert first_tokens(start_block=3) == everything[3:]
    stream = iter(TokenBinDataset(corpus_bin, max_length=16, shuffle=True, infinite=True))
    assert len([next(stream) for _ in range(2 * len(everything) + 1)]) == 2 * len(everything) + 1


def test_reader_validation(tmp_path, corpus_bin, tok):
    TokenBinDataset(corpus_bin, max_length=16, tokenizer=tok)
    wider = WordTokenizer()
    wider.add_special_tokens({"additional_special_tokens": ["<extra>"]})
    with pytest.raises(ValueError, match="vocabulary"):
        TokenBinDataset(corpus_bin, max_length=16, tokenizer=wider)
    with pytest.raises(FileNotFoundError):
        TokenBinDataset(tmp_path / "absent.bin", max_length=16)
    orphan = tmp_path / "orphan.bin"
    orphan.write_bytes(b"\0" * 64)
    with pytest.raises(FileNotFoundError, match="sidecar"):
        TokenBinDataset(orphan, max_length=16)
    with pytest.raises(ValueError, match="fewer than one block"):
        TokenBinDataset(corpus_bin, max_length=100_000)


# -- tokenizer loading -----------------------------------------------------------------------------
def test_tokenizer_source_order(monkeypatch, tmp_path):
    calls = []

    def fake_loader(identifier, **kwargs):
        calls.append((identifier, kwargs["local_files_only"]))
        if identifier == "broken/hub":
            raise OSError("offline")
        return WordTokenizer(identifier)

    monkeypatch.setattr(tokenizer_module, "_load_hf_tokenizer", fake_loader)
    local = tmp_path / "tokenizer"
    local.mkdir()
    (local / "tokenizer.json").write_text("{}")

    result = load_tokenizer(hf_name="good/hub", tokenizer_dir=local)
    assert (result.source, result.identifier) == ("hf", "good/hub")
    result = load_tokenizer(hf_name="broken/hub", tokenizer_dir=local)
    assert result.source == "local" and calls[-1] == (str(local), True)
    result = load_tokenizer(hf_name="good/hub", tokenizer_dir=local, prefer_hf=False)
    assert result.source == "local"
    result = load_tokenizer(hf_name="broken/hub", tokenizer_dir=tmp_path / "none",
                            fallback_hf_name="good/hub")
    assert result.source == "fallback_hf"
    with pytest.raises(RuntimeError, match="No tokenizer source"):
        load_tokenizer(tokenizer_dir=tmp_path / "none")
    with pytest.raises(RuntimeError, match="offline"):
        load_tokenizer(hf_name="broken/hub", tokenizer_dir=tmp_path / "none")


def test_token_bytes_table_and_cache(tmp_path, tok):
    table = get_token_bytes(tok)
    assert table.dtype == torch.int32 and table.numel() == len(tok)
    assert table[0] == 0, "special tokens weigh nothing"
    assert table[tok.get_vocab()["a"]] == 1
    assert get_token_bytes(tok, include_special=True)[0] == len("<doc>")
    cache = tmp_path / "bytes" / "table.pt"
    first = get_token_bytes(tok, cache_path=cache)
    assert cache.exists() and torch.equal(get_token_bytes(tok, cache_path=cache), first)
    with pytest.raises(ValueError, match="mismatch"):
        get_token_bytes(WordTokenizer("another"), cache_path=cache)
    with pytest.raises(ValueError, match="mismatch"):
        get_token_bytes(tok, cache_path=cache, include_special=True)


# -- streaming text ----------------------------------------------------------------------------------
@pytest.fixture()
def fake_stream(monkeypatch):
    """Replace the Hugging Face loader by an in-memory list of rows and record the call."""
    seen = {}

    class Rows(list):
        def shuffle(self, seed, buffer_size):
            return self

    def fake_load_dataset(*args, **kwargs):
        seen["args"], seen["kwargs"] = args, kwargs
        return Rows({"text": text} for text in ("ab", "cdefgh", "", "ijklmnopqrstu", "vw"))

    monkeypatch.setattr(dataset_module, "load_dataset", fake_load_dataset)
    return seen


def test_streaming_dataset_packs_shifted_blocks(fake_stream, tok):
    data = StreamingTextDataset("some/corpus", tok, split="train", max_length=4)
    stream = iter(data)
    inputs, targets = next(stream)
    joined = [0] + tok.encode("ab") + [0] + tok.encode("cdefgh")
    assert inputs.tolist() == joined[:4] and targets.tolist() == joined[1:5]
    assert fake_stream["kwargs"]["path"] == "some/corpus" and fake_stream["kwargs"]["streaming"]
    resumed = iter(StreamingTextDataset("some/corpus", tok, split="train", max_length=4, start_block=1))
    assert next(resumed)[0].tolist() == next(stream)[0].tolist()


def test_streaming_dataset_shards_by_document(fake_stream, tok):
    odd = StreamingTextDataset("c", tok, split="train", max_length=4, data_rank=1, data_world_size=2)
    inputs, _ = next(iter(odd))
    assert inputs.tolist() == ([0] + tok.encode("cdefgh"))[:4]
    for bad in (dict(data_rank=2, data_world_size=2), dict(data_rank=0), dict(start_block=-1)):
        with pytest.raises(ValueError):
            StreamingTextDataset("c", tok, split="train", max_length=4, **bad)


def test_streaming_dataset_finds_local_split_files(fake_stream, tok, tmp_path):
    (tmp_path / "train.jsonl").write_text('{"text": "x"}\n')
    (tmp_path / "validation.jsonl").write_text('{"text": "y"}\n')
    next(iter(StreamingTextDataset(str(tmp_path), tok, split="validation", max_length=4)))
    assert fake_stream["args"] == ("json",)
    assert fake_stream["kwargs"]["data_files"] == {"validation": [str(tmp_path / "validation.jsonl")]}
    with pytest.raises(FileNotFoundError):
        next(iter(StreamingTextDataset(str(tmp_path), tok, split="test", max_length=4)))


def test_dataset_module_resolves_tokenizer_names(monkeypatch):
    asked = {}

    def fake_load_tokenizer(**kwargs):
        asked.update(kwargs)
        return tokenizer_module.TokenizerLoadResult(WordTokenizer(kwargs["hf_name"]), "hf",
                                                    kwargs["hf_name"])

    monkeypatch.setattr(dataset_module, "load_tokenizer", fake_load_tokenizer)
    resolved = dataset_module.get_tokenizer("org/name")
    assert resolved.name_or_path == "org/name" and asked["prefer_hf"] is True
    assert dataset_module.get_tokenizer(None).name_or_path == dataset_module.DEFAULT_TOKENIZER
    ready = WordTokenizer()
    assert dataset_module.get_tokenizer(ready) is ready


# -- corpus staging (examples/prepare_scaling_data.py) ------------------------------------------------
def test_climbmix_defaults_and_bounds():
    staging = load_example("prepare_scaling_data")
    train, held_out = staging.nanochat_climbmix_files(3)
    assert [Path(url).name for url in train] == [f"shard_{i:05d}.parquet" for i in range(3)]
    assert held_out.endswith("shard_06542.parquet") and held_out not in train
    for count in (0, 6_543):
        with pytest.raises(ValueError):
            staging.nanochat_climbmix_files(count)


def test_stage_split_counts_tokens_and_writes_stats(tmp_path, tok):
    staging = load_example("prepare_scaling_data")
    rows = [{"text": "ab"}, {"text": ""}, {"other": 1}, {"text": "cde"}, {"text": "never reached"}]
    calls = []

    class Counting(WordTokenizer):
        def __call__(self, texts, **kwargs):
            calls.append(len(texts))
            return super().__call__(texts, **kwargs)

    done = staging.stage_split(
        dataset_name=None, dataset_config=None, source_files=None, source_split="train",
        output_split="train", text_column="text", max_documents=2, output_dir=tmp_path, force=False,
        skip_existing=False, tokenizer=Counting(), tokenizer_batch_size=1, stream=rows)
    assert (done.documents, done.utf8_bytes, done.tokens) == (2, 5, 2 + 3 + 2)
    assert calls == [1, 1]
    lines = (tmp_path / "train.jsonl").read_text().splitlines()
    assert [json.loads(line) for line in lines] == [{"text": "ab"}, {"text": "cde"}]
    assert json.loads((tmp_path / "stats.train.json").read_text())["tokens"] == 7
    common = dict(dataset_name=None, dataset_config=None, source_files=None, source_split="train",
                  output_split="train", text_column="text", max_documents=2, output_dir=tmp_path,
                  stream=rows)
    with pytest.raises(FileExistsError):
        staging.stage_split(force=False, skip_existing=False, **common)
    assert staging.stage_split(force=False, skip_existing=True, **common) is None
    with pytest.raises(ValueError, match="share a supported suffix"):
        staging.open_stream(dataset_name=None, dataset_config=None,
                            source_files=["a.parquet", "b.txt"], source_split="train")
