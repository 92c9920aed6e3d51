"""Flat pre-tokenised corpora: write once, memory-map at training time.

On-disk format (interchangeable with the reference, ohara/tokenbin.py:41-246): ``<name>.bin`` is
raw little-endian uint16 token ids with every document prefixed by the boundary token; the
``<name>.json`` sidecar records ``tokens, documents, dtype, vocab_size, tokenizer,
boundary_token_id`` so a corpus cannot be paired with the wrong vocabulary.

``TokenBinDataset`` hands out ``max_length + 1`` token blocks round-robin over the flattened
(rank, worker) grid; the block permutation is a function of ``seed + epoch`` only, so shards are
disjoint, their union covers the corpus once per epoch, and ``start_block`` gives exact resume.
"""

from __future__ import annotations

import json
from collections.abc import Iterable, Iterator
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import IterableDataset, get_worker_info

TOKEN_DTYPE = np.uint16
MAX_VOCAB = int(np.iinfo(TOKEN_DTYPE).max) + 1


def _sidecar_path(bin_path: str | Path) -> Path:
    return Path(bin_path).with_suffix(".json")


class _BinWriter:
    """Buffers encoded documents and appends them to an open file in large writes."""

    def __init__(self, handle, boundary: int, flush_every: int, progress_every: int, log: bool):
        self.handle = handle
        self.boundary = boundary
        self.flush_every = flush_every
        self.progress_every = progress_every
        self.log = log
        self.chunks: list[np.ndarray] = []
        self.buffered = 0
        self.tokens = 0
        self.documents = 0
        self._next_report = progress_every

    def add(self, encoded_batch: list[list[int]]) -> None:
        for ids in encoded_batch:
            block = np.empty(len(ids) + 1, dtype=TOKEN_DTYPE)
            block[0] = self.boundary
            block[1:] = np.asarray(ids, dtype=TOKEN_DTYPE)
            self.chunks.append(block)
            self.buffered += block.size
        self.documents += len(encoded_batch)
        if self.buffered >= self.flush_every:
            self.flush()

    def flush(self) -> None:
        if not self.chunks:
            return
        np.concatenate(self.chunks).tofile(self.handle)
        self.tokens += self.buffered
        self.chunks.clear()
        self.buffered = 0
        if self.log and self.tokens >= self._next_report:
            print(f"  {self.documents:,} docs -> {self.tokens:,} tokens", flush=True)
            self._next_report = self.tokens + self.progress_every


def write_token_bin(documents: Iterable[str], tokenizer, bin_path: str | Path, *,
                    boundary_token_id: int | None = None, batch_size: int = 1024,
                    flush_every: int = 64 * 1024 * 1024, progress_every: int = 1_000_000,
                    log: bool = True) -> dict[str, object]:
    """Tokenise ``documents`` into ``bin_path`` (+ sidecar). Non-string and empty documents are
    skipped. The file appears atomically (temp file + rename); returns the sidecar metadata."""
    if len(tokenizer) > MAX_VOCAB:
        raise ValueError(
            f"vocabulary of {len(tokenizer):,} exceeds what {TOKEN_DTYPE.__name__} can hold "
            f"({MAX_VOCAB:,}); widen TOKEN_DTYPE before using this tokenizer"
        )
    if batch_size < 1:
        raise ValueError("batch_size must be at least 1")
    if boundary_token_id is None:
        boundary_token_id = tokenizer.bos_token_id
        if boundary_token_id is None:
            boundary_token_id = tokenizer.eos_token_id
    if boundary_token_id is None:
        raise ValueError("tokenizer must define a BOS or EOS token to delimit documents")
    bin_path = Path(bin_path)
    bin_path.parent.mkdir(parents=True, exist_ok=True)
    temporary = bin_path.with_name(f".{bin_path.name}.tmp")
    try:
        with open(temporary, "wb") as handle:
            writer = _BinWriter(handle, int(boundary_token_id), flush_every, progress_every, log)
            batch: list[str] = []
            for document in documents:
                if not isinstance(document, str) or not document:
                    continue
                batch.append(document)
                if len(batch) >= batch_size:
                    writer.add(tokenizer(batch, add_special_tokens=False)["input_ids"])
                    batch = []
            if batch:
                writer.add(tokenizer(batch, add_special_tokens=False)["input_ids"])
            writer.flush()
        if writer.tokens == 0:
            raise RuntimeError("no tokens were written; the document stream was empty")
        temporary.replace(bin_path)
    finally:
        temporary.unlink(missing_ok=True)
    metadata: dict[str, object] = {
        "tokens": int(writer.tokens),
        "documents": int(writer.documents),
        "dtype": TOKEN_DTYPE.__name__,
        "vocab_size": len(tokenizer),
        "tokenizer": str(getattr(tokenizer, "name_or_path", "unknown")),
        "boundary_token_id": int(boundary_token_id),
    }
    _sidecar_path(bin_path).write_text(json.dumps(metadata, indent=2) + "\n", encoding="utf-8")
    if log:
        print(f"wrote {bin_path}: {writer.tokens:,} tokens from {writer.documents:,} documents")
    return metadata


def read_token_bin_metadata(bin_path: str | Path) -> dict[str, object]:
    sidecar = _sidecar_path(bin_path)
    if not sidecar.exists():
        raise FileNotFoundError(f"missing token-bin sidecar: {sidecar}")
    return json.loads(sidecar.read_text(encoding="utf-8"))


class TokenBinDataset(IterableDataset):
    def __init__(self, bin_path: str | Path, *, max_length: int, tokenizer=None,
                 shuffle: bool = True, seed: int = 42, infinite: bool = True, start_block: int = 0,
                 data_rank: int | None = None, data_world_size: int | None = None) -> None:
        super().__init__()
        if max_length < 2:
            raise ValueError("max_length must be at least 2")
        if start_block < 0:
            raise ValueError("start_block cannot be negative")
        if (data_rank is None) != (data_world_size is None):
            raise ValueError("data_rank and data_world_size must be provided together")
        self.bin_path = Path(bin_path)
        if not self.bin_path.exists():
            raise FileNotFoundError(f"token bin not found: {self.bin_path}")
        self.metadata = read_token_bin_metadata(self.bin_path)
        if tokenizer is not None and self.metadata["vocab_size"] != len(tokenizer):
            raise ValueError(
                f"{self.bin_path} was tokenized with a {self.metadata['vocab_size']:,} token "
                f"vocabulary but the tokenizer has {len(tokenizer):,}; re-run pretokenization"
            )
        self.max_length = max_length
        self.shuffle = shuffle
        self.seed = seed
        self.infinite = infinite
        self.start_block = start_block
        self.data_rank = data_rank
        self.data_world_size = data_world_size
        self.block_size = max_length + 1
        self.num_blocks = int(self.metadata["tokens"]) // self.block_size
        if self.num_blocks < 1:
            raise ValueError(
                f"{self.bin_path} holds {self.metadata['tokens']:,} tokens, "
                f"which is fewer than one block of {self.block_size:,}"
            )
        self._tokens: np.memmap | None = None

    def _memmap(self) -> np.memmap:
        if self._tokens is None:  # opened per worker process, never inherited across a fork
            self._tokens = np.memmap(self.bin_path, dtype=TOKEN_DTYPE, mode="r")
        return self._tokens

    def _shard(self) -> tuple[int, int]:
        worker = get_worker_info()
        worker_id, workers = (worker.id, worker.num_workers) if worker is not None else (0, 1)
        rank, world = self.data_rank, self.data_world_size
        if rank is None or world is None:
            active = dist.is_available() and dist.is_initialized()
            rank = dist.get_rank() if active else 0
            world = dist.get_world_size() if active else 1
        return rank * workers + worker_id, world * workers

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        tokens = self._memmap()
        shard, shards = self._shard()
        to_skip = self.start_block
        epoch = 0
        while True:
            order = np.arange(self.num_blocks)
            if self.shuffle:
                np.random.default_rng(self.seed + epoch).shuffle(order)
            for position in range(shard, self.num_blocks, shards):
                if to_skip > 0:
                    to_skip -= 1
                    continue
                begin = int(order[position]) * self.block_size
                block = torch.from_numpy(
                    np.asarray(tokens[begin : begin + self.block_size], dtype=np.int64)
                )
                yield block[:-1], block[1:]
            if not self.infinite:
                return
            epoch += 1
