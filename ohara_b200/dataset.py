"""Text datasets yielding ``(inputs, targets)`` LongTensors of length ``max_length``.

* ``StreamingTextDataset``: Hugging Face streaming (or local ``{split}*.{txt,json,jsonl,parquet}``)
  documents, each prefixed with the boundary token, concatenated and cut into contiguous
  ``max_length + 1`` blocks; documents are striped over the (rank, worker) grid; ``start_block``
  skips already-consumed blocks for exact resume.
* ``PreTokenizedDataset``: rows of ``input_ids`` saved with ``datasets.save_to_disk``, truncated or
  padded to ``max_length + 1``.
* ``TinyShakespeareDataset``: random windows of one small text file.

Behaviour follows the reference datasets (ohara/dataset.py:55-317). ``datasets`` is imported
lazily, inside the functions that need it.
"""

from __future__ import annotations

import os
import random
from collections.abc import Iterator
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.utils.data import IterableDataset, get_worker_info

from ohara_b200.tokenizer import load_tokenizer

PATH = Path("./data")
DEFAULT_TOKENIZER = "NeelNanda/gpt-neox-tokenizer-digits"
_LOCAL_BUILDERS = {".txt": "text", ".json": "json", ".jsonl": "json", ".parquet": "parquet"}


def load_dataset(*args, **kwargs):
    """Indirection over ``datasets.load_dataset`` (kept as a module attribute so tests can patch)."""
    import datasets

    return datasets.load_dataset(*args, **kwargs)


def load_from_disk(*args, **kwargs):
    import datasets

    return datasets.load_from_disk(*args, **kwargs)


def _resolve_tokenizer(tokenizer, *, cache_dir: str | Path | None = None):
    if tokenizer is None:
        tokenizer = DEFAULT_TOKENIZER
    if isinstance(tokenizer, str):
        tokenizer = load_tokenizer(hf_name=tokenizer, prefer_hf=True, cache_dir=cache_dir,
                                   use_fast=True).tokenizer
    if tokenizer.pad_token_id is None and tokenizer.eos_token_id is not None:
        tokenizer.pad_token = tokenizer.eos_token
    tokenizer.padding_side = "right"
    return tokenizer


def get_tokenizer(tokenizer=None, *, cache_dir: str | Path | None = None):
    """Tokenizer object from an object, a hub name or ``None`` (default tokenizer)."""
    return _resolve_tokenizer(tokenizer, cache_dir=cache_dir)


def _shard_of_process(data_rank: int | None, data_world_size: int | None) -> tuple[int, int]:
    worker = get_worker_info()
    worker_id, workers = (worker.id, worker.num_workers) if worker is not None else (0, 1)
    rank, world = data_rank, data_world_size
    if rank is None or world is None:
        active = dist.is_available() and dist.is_initialized()
        rank = dist.get_rank() if active else 0
        world = dist.get_world_size() if active else 1
    return rank * workers + worker_id, world * workers


class PreTokenizedDataset(IterableDataset):
    def __init__(self, dataset_name: str = "JeanKaddour/minipile", tokenizer=None,
                 split: str = "train", path: Path = PATH, microbatch_size: int = 32,
                 min_length: int = 512, max_length: int = 2048, hf: bool = False, cache_dir=None):
        self.tokenizer = _resolve_tokenizer(tokenizer, cache_dir=cache_dir)
        self.PAD = self.tokenizer.pad_token_id
        if self.PAD is None:
            raise ValueError("tokenizer must define a PAD or EOS token")
        self.length = self.vocab_size = len(self.tokenizer)
        self.microbatch_size = microbatch_size
        self.min_length = min_length
        self.max_length = max_length + 1
        self.cache_dir = cache_dir
        self.dataset_name = dataset_name
        location = path
        if path == PATH:
            stem = (f"{dataset_name.replace('/', '-')}--"
                    f"{self.tokenizer.name_or_path.replace('/', '-')}")
            location = str(path.joinpath(stem).joinpath(split))
        self.ds = load_dataset(dataset_name)[split] if hf else load_from_disk(location)
        if len(self.ds) == 0:
            raise ValueError(f"dataset split is empty: {location}")

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        shard, shards = _shard_of_process(None, None)
        while True:
            for index in range(shard, len(self.ds), shards):
                row = torch.tensor(self.ds[index]["input_ids"], dtype=torch.long)[: self.max_length]
                row = F.pad(row, (0, self.max_length - row.shape[0]), "constant", value=self.PAD)
                yield row[:-1], row[1:]


class StreamingTextDataset(IterableDataset):
    def __init__(self, dataset_name: str, tokenizer, *, split: str, max_length: int,
                 name: str | None = None, text_column: str = "text", shuffle: bool = False,
                 shuffle_buffer_size: int = 1_000, seed: int = 42,
                 cache_dir: str | Path | None = None, data_rank: int | None = None,
                 data_world_size: int | None = None, start_block: int = 0) -> None:
        super().__init__()
        if max_length < 2:
            raise ValueError("max_length must be at least 2")
        if shuffle_buffer_size < 1:
            raise ValueError("shuffle_buffer_size must be at least 1")
        if (data_rank is None) != (data_world_size is None):
            raise ValueError("data_rank and data_world_size must be provided together")
        if data_world_size is not None and data_world_size < 1:
            raise ValueError("data_world_size must be at least 1")
        if data_rank is not None and not 0 <= data_rank < data_world_size:
            raise ValueError("data_rank must be between 0 and data_world_size - 1")
        if start_block < 0:
            raise ValueError("start_block cannot be negative")
        self.dataset_name = dataset_name
        self.name = name
        self.split = split
        self.max_length = max_length
        self.text_column = text_column
        self.shuffle = shuffle
        self.shuffle_buffer_size = shuffle_buffer_size
        self.seed = seed
        self.cache_dir = cache_dir
        self.data_rank = data_rank
        self.data_world_size = data_world_size
        self.start_block = start_block
        self.tokenizer = _resolve_tokenizer(tokenizer, cache_dir=cache_dir)
        boundary = self.tokenizer.bos_token_id
        if boundary is None:
            boundary = self.tokenizer.eos_token_id
        if boundary is None:
            raise ValueError("tokenizer must define a BOS or EOS token for document boundaries")
        self.boundary_token_id = boundary

    def _load_stream(self):
        local = Path(self.dataset_name).expanduser()
        if local.exists():
            if local.is_file():
                builder = _LOCAL_BUILDERS.get(local.suffix.lower())
                if builder is None:
                    raise ValueError(f"unsupported local dataset file: {local}")
                files: str | list[str] = str(local)
            else:
                builder, files = None, []
                for suffix, candidate in _LOCAL_BUILDERS.items():
                    found = sorted(local.glob(f"{self.split}*{suffix}"))
                    if found:
                        builder, files = candidate, [str(p) for p in found]
                        break
                if builder is None:
                    raise FileNotFoundError(
                        f"no {self.split!r} text, JSONL, JSON, or Parquet files in {local}"
                    )
            return load_dataset(builder, data_files={self.split: files}, split=self.split,
                                streaming=True, cache_dir=self.cache_dir)
        kwargs = {"path": self.dataset_name, "split": self.split, "streaming": True,
                  "cache_dir": self.cache_dir}
        if self.name is not None:
            kwargs["name"] = self.name
        return load_dataset(**kwargs)

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        shard, shards = _shard_of_process(self.data_rank, self.data_world_size)
        base = self._load_stream()
        block_size = self.max_length + 1
        tokens: list[int] = []
        head = 0  # index of the first unconsumed token in `tokens`
        to_skip = self.start_block
        epoch = 0
        while True:
            stream = base
            if self.shuffle:
                stream = stream.shuffle(seed=self.seed + epoch, buffer_size=self.shuffle_buffer_size)
            saw_document = False
            for index, row in enumerate(stream):
                if index % shards != shard:
                    continue
                if self.text_column not in row:
                    raise KeyError(f"dataset row does not contain text column {self.text_column!r}")
                text = row[self.text_column]
                if not isinstance(text, str) or not text:
                    continue
                saw_document = True
                tokens.append(self.boundary_token_id)
                tokens.extend(self.tokenizer.encode(text, add_special_tokens=False))
                while len(tokens) - head >= block_size:
                    block = torch.tensor(tokens[head : head + block_size], dtype=torch.long)
                    head += block_size
                    if to_skip > 0:
                        to_skip -= 1
                    else:
                        yield block[:-1], block[1:]
                if head >= block_size * 16:
                    tokens = tokens[head:]
                    head = 0
            if not saw_document:
                raise RuntimeError(
                    f"no usable documents found in {self.dataset_name!r} split {self.split!r}"
                )
            epoch += 1


class TinyShakespeareDataset(IterableDataset):
    URL = "https://raw.githubusercontent.com/karpathy/char-rnn/master/data/tinyshakespeare/input.txt"

    def __init__(self, tokenizer=None, path: Path = PATH, min_length: int = 512,
                 max_length: int = 512, cache_dir=None):
        self.tokenizer = _resolve_tokenizer(tokenizer, cache_dir=cache_dir)
        self.PAD = self.tokenizer.pad_token_id
        self.vocab_size = len(self.tokenizer)
        self.min_length = min_length
        self.max_length = max_length
        self.cache_dir = cache_dir
        self.dataset_name = "tinyshakespeare"
        self.data_path = Path(path).joinpath(self.dataset_name + ".txt")
        if not self.data_path.exists():
            self.download_data()
        text = self.data_path.read_text(encoding="utf-8")
        self.data = torch.tensor(self.tokenizer.encode(text), dtype=torch.long)
        self.length = len(self.data)

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        while True:
            start = random.randint(0, self.length - self.max_length - 1)
            window = self.data[start : start + self.max_length + 1]
            yield window[:-1], window[1:]

    def download_data(self) -> None:
        import requests

        response = requests.get(self.URL)
        if response.status_code != 200:
            raise RuntimeError(f"Failed to download data. Status code: {response.status_code}")
        os.makedirs(self.data_path.parent, exist_ok=True)
        self.data_path.write_text(response.text, encoding="utf-8")
