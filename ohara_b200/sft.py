"""Supervised-finetuning data: conversation sources and best-fit packed, masked rows.

Conversations are indivisible, so rows are *packed*, never cut from a continuous stream: each row
of ``max_length + 1`` tokens is filled by repeatedly taking the longest buffered conversation that
still fits (best fit over a lookahead buffer); when nothing fits the tail is padded. Padding and
every non-assistant token carry ``ignore_index`` targets. Behaviour follows the reference packer
(ohara/sft.py:234-382) and sources (ohara/sft.py:54-227).
"""

from __future__ import annotations

import random
import re
from collections.abc import Callable, Iterator, Sequence
from typing import Any

import torch
import torch.distributed as dist
from torch.utils.data import IterableDataset, get_worker_info

from ohara_b200.chat import IGNORE_INDEX, render_conversation

Conversation = dict[str, Any]
ConversationSource = Callable[[], Sequence[Conversation]]

MC_LETTERS = ("A", "B", "C", "D")


# --------------------------------------------------------------------------------------------------
# Sources (Hugging Face datasets, loaded eagerly: the mixture is small and gets shuffled)
# --------------------------------------------------------------------------------------------------
def _load(dataset_name: str, config: str | None, split: str, cache_dir: str | None):
    from datasets import load_dataset

    kwargs: dict[str, Any] = {"path": dataset_name, "split": split, "cache_dir": cache_dir}
    if config is not None:
        kwargs["name"] = config
    return load_dataset(**kwargs)


def _take(rows, convert, limit: int | None) -> list[Conversation]:
    out: list[Conversation] = []
    for row in rows:
        conversation = convert(row)
        if conversation is None:
            continue
        out.append(conversation)
        if limit is not None and len(out) >= limit:
            break
    return out


def smoltalk_conversations(split: str = "train", *, limit: int | None = None,
                           cache_dir: str | None = None) -> list[Conversation]:
    """General chat data from ``HuggingFaceTB/smol-smoltalk``."""
    if split not in {"train", "test"}:
        raise ValueError("smoltalk split must be 'train' or 'test'")

    def convert(row):
        if len(row["messages"]) < 2:
            return None
        return {"messages": [dict(m) for m in row["messages"]]}

    return _take(_load("HuggingFaceTB/smol-smoltalk", None, split, cache_dir), convert, limit)


_GSM8K_TOOL_CALL = re.compile(r"(<<[^>]+>>)")


def gsm8k_answer_parts(answer: str) -> list[dict[str, str]]:
    """Split a GSM8K solution into text / python / python_output parts at ``<<expr=result>>``."""
    parts: list[dict[str, str]] = []
    for chunk in _GSM8K_TOOL_CALL.split(answer):
        if chunk.startswith("<<") and chunk.endswith(">>"):
            expression, _, result = chunk[2:-2].rpartition("=")
            if not expression:
                expression, result = chunk[2:-2], ""
            parts.append({"type": "python", "text": expression})
            parts.append({"type": "python_output", "text": result})
        elif chunk:
            parts.append({"type": "text", "text": chunk})
    return parts


def gsm8k_conversations(split: str = "train", *, limit: int | None = None,
                        cache_dir: str | None = None,
                        use_tool_calls: bool = True) -> list[Conversation]:
    """Grade-school maths; calculator annotations become tool-call parts (or are stripped)."""
    if split not in {"train", "test"}:
        raise ValueError("gsm8k split must be 'train' or 'test'")

    def convert(row):
        answer = row["answer"]
        content: Any = gsm8k_answer_parts(answer) if use_tool_calls else _GSM8K_TOOL_CALL.sub("", answer)
        return {"messages": [{"role": "user", "content": row["question"]},
                             {"role": "assistant", "content": content}]}

    return _take(_load("openai/gsm8k", "main", split, cache_dir), convert, limit)


def render_multiple_choice(question: str, choices: Sequence[str]) -> str:
    """Multiple-choice prompt with the letter *after* each choice and no space before it, so the
    prompt's letter token equals the one the assistant must emit."""
    lines = "".join(f"- {choice}={letter}\n" for letter, choice in zip(MC_LETTERS, choices))
    return (f"Multiple Choice question: {question}\n{lines}\n"
            "Respond only with the letter of the correct answer.")


def mmlu_conversations(split: str = "auxiliary_train", *, limit: int | None = None,
                       cache_dir: str | None = None) -> list[Conversation]:
    valid = {"auxiliary_train", "validation", "dev", "test"}
    if split not in valid:
        raise ValueError(f"mmlu split must be one of {sorted(valid)}")

    def convert(row):
        if len(row["choices"]) != len(MC_LETTERS):
            return None
        return {"messages": [
            {"role": "user", "content": render_multiple_choice(row["question"], row["choices"])},
            {"role": "assistant", "content": MC_LETTERS[int(row["answer"])]},
        ]}

    return _take(_load("cais/mmlu", "all", split, cache_dir), convert, limit)


def build_mixture(*, split: str = "train", smoltalk_limit: int | None = None, mmlu_epochs: int = 1,
                  mmlu_limit: int | None = None, gsm8k_epochs: int = 1,
                  gsm8k_limit: int | None = None, cache_dir: str | None = None,
                  seed: int = 42) -> list[Conversation]:
    """SmolTalk + MMLU + GSM8K, shuffled with ``seed``; ``*_epochs`` repeats the small sources."""
    if split not in {"train", "val"}:
        raise ValueError("mixture split must be 'train' or 'val'")
    if mmlu_epochs < 0 or gsm8k_epochs < 0:
        raise ValueError("epoch counts cannot be negative")
    mix: list[Conversation] = []
    if split == "train":
        mix += smoltalk_conversations("train", limit=smoltalk_limit, cache_dir=cache_dir)
        for _ in range(mmlu_epochs):
            mix += mmlu_conversations("auxiliary_train", limit=mmlu_limit, cache_dir=cache_dir)
        for _ in range(gsm8k_epochs):
            mix += gsm8k_conversations("train", limit=gsm8k_limit, cache_dir=cache_dir)
    else:
        mix += smoltalk_conversations("test", limit=smoltalk_limit, cache_dir=cache_dir)
        mix += mmlu_conversations("test", limit=mmlu_limit or 5_200, cache_dir=cache_dir)
        mix += gsm8k_conversations("test", limit=gsm8k_limit or 420, cache_dir=cache_dir)
    if not mix:
        raise RuntimeError(f"SFT {split} mixture is empty")
    random.Random(seed).shuffle(mix)
    return mix


# --------------------------------------------------------------------------------------------------
# Packing
# --------------------------------------------------------------------------------------------------
class BestFitPacker:
    """Packs ``(ids, mask)`` items into rows of ``capacity`` tokens using a lookahead buffer."""

    def __init__(self, capacity: int, buffer_size: int, pad_token_id: int) -> None:
        self.capacity = capacity
        self.buffer_size = buffer_size
        self.pad_token_id = pad_token_id

    def rows(self, items: Iterator[tuple[list[int], list[int]]]) -> Iterator[tuple[list[int], list[int]]]:
        pending: list[tuple[list[int], list[int]]] = []
        drained = False

        def refill() -> None:
            nonlocal drained
            while not drained and len(pending) < self.buffer_size:
                try:
                    pending.append(next(items))
                except StopIteration:
                    drained = True

        while True:
            refill()
            if not pending:
                return
            ids: list[int] = []
            mask: list[int] = []
            while pending:
                room = self.capacity - len(ids)
                pick, pick_len = -1, -1
                for index, (candidate, _) in enumerate(pending):
                    if pick_len < len(candidate) <= room:
                        pick, pick_len = index, len(candidate)
                if pick < 0:
                    break
                chosen_ids, chosen_mask = pending.pop(pick)
                ids += chosen_ids
                mask += chosen_mask
                refill()
            if not ids:
                raise RuntimeError("conversation does not fit in a single row")
            pad = self.capacity - len(ids)
            if pad:
                ids += [self.pad_token_id] * pad
                mask += [0] * pad
            yield ids, mask


class ConversationDataset(IterableDataset):
    """Yields ``(inputs, targets)`` LongTensors of length ``max_length`` for the trainer."""

    def __init__(self, conversations: Sequence[Conversation], tokenizer, *, max_length: int,
                 buffer_size: int = 100, ignore_index: int = IGNORE_INDEX, seed: int = 42,
                 shuffle: bool = True, infinite: bool = True, data_rank: int | None = None,
                 data_world_size: int | None = None) -> None:
        super().__init__()
        if max_length < 2:
            raise ValueError("max_length must be at least 2")
        if buffer_size < 1:
            raise ValueError("buffer_size must be at least 1")
        if not conversations:
            raise ValueError("conversations must not be empty")
        if (data_rank is None) != (data_world_size is None):
            raise ValueError("data_rank and data_world_size must be provided together")
        self.conversations = conversations
        self.tokenizer = tokenizer
        self.max_length = max_length
        self.buffer_size = buffer_size
        self.ignore_index = ignore_index
        self.seed = seed
        self.shuffle = shuffle
        self.infinite = infinite
        self.data_rank = data_rank
        self.data_world_size = data_world_size
        self.row_capacity = max_length + 1  # the shift into (inputs, targets) consumes one token
        pad = tokenizer.pad_token_id
        if pad is None:
            pad = tokenizer.eos_token_id
        if pad is None:
            raise ValueError("tokenizer must define a PAD or EOS token for padding")
        self.pad_token_id = pad

    def _shard(self) -> tuple[int, int]:
        worker = get_worker_info()
        worker_id, workers = (worker.id, worker.num_workers) if worker is not None else (0, 1)
        rank, world = self.data_rank, self.data_world_size
        if rank is None or world is None:
            active = dist.is_available() and dist.is_initialized()
            rank = dist.get_rank() if active else 0
            world = dist.get_world_size() if active else 1
        return rank * workers + worker_id, world * workers

    def _rendered(self, epoch: int) -> Iterator[tuple[list[int], list[int]]]:
        """This shard's conversations as ``(ids, mask)``; malformed or unsupervised ones skipped."""
        shard, shards = self._shard()
        order = list(range(len(self.conversations)))
        if self.shuffle:
            random.Random(self.seed + epoch).shuffle(order)
        for position, index in enumerate(order):
            if position % shards != shard:
                continue
            try:
                ids, mask = render_conversation(
                    self.tokenizer, self.conversations[index]["messages"],
                    max_tokens=self.row_capacity,
                )
            except ValueError:
                continue
            if len(ids) < 2 or not any(mask):
                continue
            yield ids, mask

    def __iter__(self) -> Iterator[tuple[torch.Tensor, torch.Tensor]]:
        packer = BestFitPacker(self.row_capacity, self.buffer_size, self.pad_token_id)
        epoch = 0
        while True:
            for ids, mask in packer.rows(self._rendered(epoch)):
                row = torch.tensor(ids, dtype=torch.long)
                keep = torch.tensor(mask[1:], dtype=torch.bool)
                targets = torch.where(keep, row[1:], torch.full_like(row[1:], self.ignore_index))
                yield row[:-1].clone(), targets
            if not self.infinite:
                return
            epoch += 1
