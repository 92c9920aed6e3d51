"""Phi-2 in the shape of the ``microsoft/phi-2`` checkpoint: attention and MLP run in parallel off
one LayerNorm, RoPE rotates only ``rotary_dim`` of each head (half-split pairs), attention math in
fp32, KV cache for decoding, and ``from_pretrained`` maps Hugging Face safetensors shards onto
these parameter names. Reference: ohara/models/phi.py:23-256."""

from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200.embeddings_pos.rotary import RoPE
from ohara_b200.modules.kv_cache import KVCache
from ohara_b200.modules.mlp import Linear


@dataclass
class PhiConfig:
    vocab_size: int = 51200
    max_sequence_length: int = 2048
    hidden_size: int = 2560
    num_attention_heads: int = 32
    num_hidden_layers: int = 32
    dropout: float = 0.2
    multiple_of: int = 4
    bias: bool = True
    eps: float = 1e-5
    rotary_dim: float = 0.4


def new_gelu(x: Tensor) -> Tensor:
    """tanh approximation of GELU, as used by the original checkpoint."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3.0))))


class MLP(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1 = Linear(dim, hidden)
        self.fc2 = Linear(hidden, dim)

    def forward(self, x: Tensor) -> Tensor:
        return self.fc2(new_gelu(self.fc1(x)))


class PhiMHA(nn.Module):
    def __init__(self, layer_idx, hidden_size: int, num_attention_heads: int, rotary_dim: float):
        super().__init__()
        self.hidden_size = hidden_size
        self.num_attention_heads = num_attention_heads
        self.head_dim = hidden_size // num_attention_heads
        self.layer_idx = layer_idx
        self.k_proj = Linear(hidden_size, hidden_size)
        self.q_proj = Linear(hidden_size, hidden_size)
        self.v_proj = Linear(hidden_size, hidden_size)
        self.dense = Linear(hidden_size, hidden_size)
        self.rope = RoPE(int(rotary_dim * self.head_dim), traditional=False)

    def forward(self, x: Tensor, mask: Tensor | None = None, kv_cache: KVCache | None = None,
                position_ids: int | None = None) -> Tensor:
        batch, seq, _ = x.shape
        split = (batch, seq, self.num_attention_heads, self.head_dim)
        q, k, v = self.q_proj(x).view(split), self.k_proj(x).view(split), self.v_proj(x).view(split)
        start = 0
        if kv_cache is not None:
            if position_ids is None:
                raise ValueError("position_ids is required when using a KV cache")
            start = int(position_ids)
            k, v = kv_cache.forward(k, v, start)
        # Unrotated keys are cached; rotation is applied to the whole key history every step.
        q = self.rope(q.transpose(1, 2).float(), offset=start)
        k = self.rope(k.transpose(1, 2).float())
        v = v.transpose(1, 2).float()
        scores = (q @ k.transpose(-1, -2)) * math.sqrt(1 / q.shape[-1])
        q_pos = start + torch.arange(seq, device=x.device)
        k_pos = torch.arange(k.size(2), device=x.device)
        scores = scores.masked_fill(~(k_pos[None, :] <= q_pos[:, None]), float("-inf"))
        out = (torch.softmax(scores, dim=-1) @ v).type_as(x)
        return self.dense(out.transpose(1, 2).reshape(batch, seq, self.hidden_size))


class Block(nn.Module):
    def __init__(self, config: PhiConfig, block_idx: int | None = None) -> None:
        super().__init__()
        self.ln = nn.LayerNorm(config.hidden_size, eps=config.eps)
        self.block_idx = block_idx
        self.mixer = PhiMHA(block_idx, config.hidden_size, config.num_attention_heads,
                            config.rotary_dim)
        self.mlp = MLP(config.hidden_size, config.multiple_of * config.hidden_size)

    def forward(self, x: Tensor, mask: Tensor | None = None, kv_cache: KVCache | None = None,
                position_ids: int | None = None) -> Tensor:
        h = self.ln(x)
        return self.mixer(h, mask, kv_cache, position_ids) + self.mlp(h) + x


class Phi(nn.Module):
    def __init__(self, config: PhiConfig) -> None:
        super().__init__()
        self.config = config
        self.wte = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([Block(config, i) for i in range(config.num_hidden_layers)])
        self.ln = nn.LayerNorm(config.hidden_size, eps=config.eps)
        self.lm_head = Linear(config.hidden_size, config.vocab_size)
        self.loss_fn = nn.CrossEntropyLoss()
        self.mask = None  # causal masking is computed from positions inside the mixer

    def forward(self, x: Tensor, kv_cache: list[KVCache] | None = None,
                position_ids: int | None = None) -> Tensor:
        """``x`` holds only the tokens not yet in the cache."""
        if kv_cache is not None and len(kv_cache) != len(self.layers):
            raise ValueError("KV cache must contain one entry per model layer")
        h = self.wte(x).to(self.wte.weight.dtype)
        for idx, layer in enumerate(self.layers):
            h = layer(h, self.mask, kv_cache[idx] if kv_cache is not None else None,
                      position_ids=position_ids)
        return self.lm_head(self.ln(h))

    def loss(self, logits: Tensor, labels: Tensor) -> Tensor:
        return self.loss_fn(logits.view(-1, logits.size(-1)), labels.view(-1))

    def build_kv_cache(self, batch_size: int = 1) -> list[KVCache]:
        if batch_size < 1:
            raise ValueError("batch_size must be at least 1")
        cfg = self.config
        shape = (batch_size, cfg.max_sequence_length, cfg.num_attention_heads,
                 cfg.hidden_size // cfg.num_attention_heads)
        weight = self.wte.weight
        return [KVCache(shape, cfg.max_sequence_length, idx, device=weight.device, dtype=weight.dtype)
                for idx in range(cfg.num_hidden_layers)]

    @staticmethod
    def _huggingface_state_dict_map(num_hidden_layers: int) -> dict[str, str]:
        """This implementation's parameter names → ``microsoft/phi-2`` names."""
        names = {
            "wte.weight": "model.embed_tokens.weight",
            "ln.weight": "model.final_layernorm.weight",
            "ln.bias": "model.final_layernorm.bias",
            "lm_head.weight": "lm_head.weight",
            "lm_head.bias": "lm_head.bias",
        }
        for idx in range(num_hidden_layers):
            for kind in ("weight", "bias"):
                names[f"layers.{idx}.ln.{kind}"] = f"model.layers.{idx}.input_layernorm.{kind}"
                for fc in ("fc1", "fc2"):
                    names[f"layers.{idx}.mlp.{fc}.{kind}"] = f"model.layers.{idx}.mlp.{fc}.{kind}"
                for proj in ("q_proj", "k_proj", "v_proj", "dense"):
                    names[f"layers.{idx}.mixer.{proj}.{kind}"] = (
                        f"model.layers.{idx}.self_attn.{proj}.{kind}")
        return names

    @classmethod
    def from_pretrained(cls, name: str) -> "Phi":
        """Download ``name`` from the Hub and load it into an fp16 model."""
        from safetensors import safe_open

        from ohara_b200.utils.load import download_hf_model

        config = PhiConfig()
        model = cls(config).half()
        folder = Path(download_hf_model(name))
        tensors: dict[str, Tensor] = {}
        for shard in sorted(folder.glob("*.safetensors")):
            with safe_open(shard, framework="pt", device="cpu") as reader:
                for key in reader.keys():
                    tensors[key] = reader.get_tensor(key)
        if not tensors:
            raise FileNotFoundError(f"no safetensors shards found in {folder}")
        names = cls._huggingface_state_dict_map(config.num_hidden_layers)
        missing = sorted(set(names.values()) - set(tensors))
        if missing:
            raise KeyError(f"checkpoint is missing expected tensors: {missing[:5]}")
        model.load_state_dict({ours: tensors[theirs] for ours, theirs in names.items()}, strict=True)
        return model
