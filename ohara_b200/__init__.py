"""ohara_b200: a Blackwell-native LLM training and chat framework.

Same public names as the ``ohara`` package it can replace (``Config``, ``Llama``, ``Trainer``,
``OharaEngine`` and its config/enum types, ``ChatEngine``, ``SamplingConfig``,
``ConversationDataset``, ``load_chat_tokenizer``, ``render_conversation``, the schedulers and the
datasets), resolved lazily so that ``import ohara_b200`` costs no more than ``import torch``. The
hot ops underneath are hand-written sm_100a kernels (``ohara_b200/csrc``), reached through
``ohara_b200.ops``.
"""

from __future__ import annotations

import importlib
from typing import TYPE_CHECKING

__version__ = "0.1.0"

_EXPORTS = {
    "Config": "ohara_b200.models.llama",
    "Llama": "ohara_b200.models.llama",
    "PreTokenizedDataset": "ohara_b200.dataset",
    "StreamingTextDataset": "ohara_b200.dataset",
    "TinyShakespeareDataset": "ohara_b200.dataset",
    "ChatEngine": "ohara_b200.chat_engine",
    "ConversationDataset": "ohara_b200.sft",
    "SamplingConfig": "ohara_b200.chat_engine",
    "load_chat_tokenizer": "ohara_b200.chat",
    "render_conversation": "ohara_b200.chat",
    "CosineScheduler": "ohara_b200.lr_scheduler",
    "Scheduler": "ohara_b200.lr_scheduler",
    "Trainer": "ohara_b200.trainer",
    "Backend": "ohara_b200.runtime",
    "DistributedConfig": "ohara_b200.runtime",
    "EngineConfig": "ohara_b200.runtime",
    "OharaEngine": "ohara_b200.runtime",
    "ParallelConfig": "ohara_b200.runtime",
    "PipelinePlan": "ohara_b200.runtime",
    "PipelineScheduleType": "ohara_b200.runtime",
    "PipelineStageSpec": "ohara_b200.runtime",
    "PrecisionConfig": "ohara_b200.runtime",
    "PrecisionMode": "ohara_b200.runtime",
    "ReduceType": "ohara_b200.runtime",
    "StrategyType": "ohara_b200.runtime",
    "TensorParallelPlan": "ohara_b200.runtime",
    "TensorParallelRule": "ohara_b200.runtime",
    "TensorParallelStyle": "ohara_b200.runtime",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str):
    target = _EXPORTS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(target), name)
    globals()[name] = value
    return value


def __dir__() -> list[str]:
    return __all__


if TYPE_CHECKING:  # pragma: no cover
    from .chat import load_chat_tokenizer, render_conversation  # noqa: F401
    from .chat_engine import ChatEngine, SamplingConfig  # noqa: F401
    from .dataset import (  # noqa: F401
        PreTokenizedDataset,
        StreamingTextDataset,
        TinyShakespeareDataset,
    )
    from .lr_scheduler import CosineScheduler, Scheduler  # noqa: F401
    from .models.llama import Config, Llama  # noqa: F401
    from .runtime import (  # noqa: F401
        Backend,
        DistributedConfig,
        EngineConfig,
        OharaEngine,
        ParallelConfig,
        PipelinePlan,
        PipelineScheduleType,
        PipelineStageSpec,
        PrecisionConfig,
        PrecisionMode,
        ReduceType,
        StrategyType,
        TensorParallelPlan,
        TensorParallelRule,
        TensorParallelStyle,
    )
    from .sft import ConversationDataset  # noqa: F401
    from .trainer import Trainer  # noqa: F401
