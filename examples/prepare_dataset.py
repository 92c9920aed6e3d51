"""Download a dataset and pretokenise it to ``./data`` for ``PreTokenizedDataset``.

    python examples/prepare_dataset.py tinystories
    python examples/prepare_dataset.py fineweb-edu --push --hf-username you

Recipes follow the reference entry point (examples/prepare_dataset.py:33-56).
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path
from typing import NamedTuple

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # run from a source checkout

from ohara_b200.pretokenize import DatasetPreprocessor, OpenHermesDatasetPreprocessor

HF_CACHE = Path("./hf_cache")


class Recipe(NamedTuple):
    dataset: str
    tokenizer: str
    splits: tuple[str, ...] = ("train", "validation")
    name: str | None = None
    revision: str | None = None
    preprocessor: type[DatasetPreprocessor] = DatasetPreprocessor


RECIPES = {
    "tinystories": Recipe("roneneldan/TinyStories", "microsoft/phi-2"),
    "minipile": Recipe("JeanKaddour/minipile", "EleutherAI/gpt-neo-125m"),
    "fineweb-edu": Recipe("HuggingFaceFW/fineweb-edu", "EleutherAI/gpt-neo-125m", name="sample-10BT"),
    "openhermes": Recipe("teknium/OpenHermes-2.5", "philschmid/gemma-tokenizer-chatml",
                         splits=("train",), revision="f7e624a58ce3642ec50483cb6039468ee8c3c464",
                         preprocessor=OpenHermesDatasetPreprocessor),
}


def main() -> None:
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("recipe", choices=sorted(RECIPES))
    p.add_argument("--tokenizer", default=None, help="override the recipe's tokenizer")
    p.add_argument("--push", action="store_true", help="also push the result to the Hub")
    p.add_argument("--hf-username", default=None)
    p.add_argument("--num-proc", type=int, default=1)
    args = p.parse_args()
    if args.push and not args.hf_username:
        raise SystemExit("--push requires --hf-username")
    recipe = RECIPES[args.recipe]
    tokenizer = args.tokenizer or recipe.tokenizer
    print(f"Pretokenizing dataset={recipe.dataset!r} with tokenizer={tokenizer!r}")
    worker = recipe.preprocessor(dataset_name=recipe.dataset, tokenizer_name=tokenizer,
                                 splits=list(recipe.splits), name=recipe.name,
                                 revision=recipe.revision, hf_cache=HF_CACHE, num_proc=args.num_proc)
    worker.process_and_save(push=args.push, hf_username=args.hf_username)


if __name__ == "__main__":
    main()
