"""Offline pre-tokenisation of Hugging Face text datasets to ``datasets`` on-disk format
(consumed by :class:`ohara_b200.dataset.PreTokenizedDataset`). Reference:
ohara/pretokenize.py:12-145."""

from __future__ import annotations

import os
from pathlib import Path

from ohara_b200.tokenizer import get_tokenizer


class DatasetPreprocessor:
    """Tokenise → shuffle → drop rows shorter than ``min_length`` → save (and optionally push)."""

    shuffle_seed = 31415

    def __init__(self, dataset_name: str = "JeanKaddour/minipile",
                 tokenizer_name: str = "NeelNanda/gpt-neox-tokenizer-digits",
                 name: str | None = None, min_length: int = 512, max_length: int = 2049,
                 splits: list[str] | None = None, revision: str | None = None,
                 num_proc: int | None = None, output_dir: Path = Path("./data"),
                 hf_cache: Path = Path("./hf_cache")):
        self.dataset_name = dataset_name
        self.tokenizer_name = tokenizer_name
        self.name = name
        self.min_length = min_length
        self.max_length = max_length
        self.splits = splits if splits is not None else ["train", "test"]
        self.output_dir = Path(output_dir)
        self.hf_cache = hf_cache
        self.revision = revision
        self.tokenizer = get_tokenizer(hf_name=tokenizer_name, prefer_hf=True, cache_dir=hf_cache)
        self.tokenizer.padding_side = "right"
        self.PAD = self.tokenizer.pad_token_id
        self.length = self.tokenizer.vocab_size
        self.num_proc = num_proc if num_proc else max((os.cpu_count() or 4) - 3, 1)

    # -- hooks ---------------------------------------------------------------------------------
    def tokenize_fn(self, x):
        return self.tokenizer(x["text"], max_length=self.max_length, truncation=True)

    def filter_fn(self, x) -> bool:
        return len(x["input_ids"]) >= self.min_length

    def _storage_name(self) -> str:
        return (f"{self.dataset_name.replace('/', '-')}--"
                f"{self.tokenizer.name_or_path.replace('/', '-')}")

    # -- pipeline ------------------------------------------------------------------------------
    def _load(self, split: str, **extra):
        from datasets import DownloadMode, load_dataset

        return load_dataset(self.dataset_name, split=split,
                            download_mode=DownloadMode.REUSE_CACHE_IF_EXISTS,
                            revision=self.revision, **extra)

    def load_and_preprocess_dataset(self, split, remove_columns=("text",)):
        dataset = self._load(split, name=self.name, cache_dir=self.hf_cache)
        return (
            dataset.map(self.tokenize_fn, batched=True, remove_columns=list(remove_columns),
                        num_proc=self.num_proc)
            .shuffle(seed=self.shuffle_seed)
            .filter(self.filter_fn, num_proc=self.num_proc)
        )

    def save_pre_tokenized_dataset(self, dataset, split) -> None:
        self.output_dir.mkdir(parents=True, exist_ok=True)
        dataset.save_to_disk(str(self.output_dir / self._storage_name() / split))
        print(f"Dataset saved to {self.output_dir}")

    def push_pre_tokenized_dataset(self, dataset, split, hf_username) -> None:
        repo = (f"{hf_username}/pretokenized__{self.dataset_name.replace('/', '_')}__"
                f"{self.tokenizer.name_or_path.replace('/', '__')}")
        dataset.push_to_hub(repo, split=split)
        print(f"Dataset pushed to hf {repo}")

    def process_and_save(self, remove_columns=("text",), push: bool = False, hf_username=None) -> None:
        for split in self.splits:
            dataset = self.load_and_preprocess_dataset(split, remove_columns=remove_columns)
            self.save_pre_tokenized_dataset(dataset, split)
            print(f"{split} Processing and saving completed.")
            if push:
                assert hf_username is not None
                self.push_pre_tokenized_dataset(dataset, split, hf_username)


class OpenHermesDatasetPreprocessor(DatasetPreprocessor):
    """OpenHermes conversations rendered through the tokenizer's chat template; rows must fit
    ``[min_length, max_length]``."""

    shuffle_seed = 42
    _ROLES = {"system": "system", "gpt": "assistant", "human": "user"}

    def load_and_preprocess_dataset(self, split, remove_columns=("text",)):
        def to_chat(item):
            turns = [{"role": self._ROLES[t["from"]], "content": t["value"]}
                     for t in item["conversations"] if t["from"] in self._ROLES]
            return {"input_ids": self.tokenizer.apply_chat_template(turns)}

        return (self._load(split).map(to_chat, num_proc=self.num_proc)
                .shuffle(seed=self.shuffle_seed).filter(self.filter_fn, num_proc=self.num_proc))

    def filter_fn(self, x) -> bool:
        return self.min_length <= len(x["input_ids"]) <= self.max_length
