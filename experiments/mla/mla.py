"""Multi-head latent attention (DeepSeek-V2; reference: experiments/MLA/mla.py:65-232).

Queries and keys/values are produced through low-rank bottlenecks (``q_lora_rank``,
``kv_lora_rank``) with an RMSNorm on the compressed vector. A head's query / key is the
concatenation of a position-free part (``nope_head_dim``) and a rotary part (``rope_head_dim``);
the rotary key is a single head shared by all query heads. The value head size may differ from the
query / key head size.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.embeddings_pos.rotary import apply_rope, precompute_freqs_cis
from ohara_b200.modules.norm import RMSNorm


@dataclass
class MLAConfig:
    d_model: int = 256
    num_heads: int = 4
    v_head_dim: int = 32
    nope_head_dim: int = 32
    rope_head_dim: int = 16
    q_lora_rank: int = 64
    kv_lora_rank: int = 64
    dropout: float = 0.0
    max_sequence_length: int = 256
    rope_theta: float = 10000.0


class MultiHeadLatentAttention(nn.Module):
    def __init__(self, cfg: MLAConfig) -> None:
        super().__init__()
        self.cfg = cfg
        h = cfg.num_heads
        self.compress_q = nn.Linear(cfg.d_model, cfg.q_lora_rank, bias=False)
        self.q_norm = RMSNorm(cfg.q_lora_rank)
        self.q_nope = nn.Linear(cfg.q_lora_rank, h * cfg.nope_head_dim, bias=False)
        self.q_rope = nn.Linear(cfg.q_lora_rank, h * cfg.rope_head_dim, bias=False)
        self.compress_kv = nn.Linear(cfg.d_model, cfg.kv_lora_rank, bias=False)
        self.kv_norm = RMSNorm(cfg.kv_lora_rank)
        self.k_nope = nn.Linear(cfg.kv_lora_rank, h * cfg.nope_head_dim, bias=False)
        self.value = nn.Linear(cfg.kv_lora_rank, h * cfg.v_head_dim, bias=False)
        self.k_rope = nn.Linear(cfg.d_model, cfg.rope_head_dim, bias=False)  # one shared head
        self.proj = nn.Linear(h * cfg.v_head_dim, cfg.d_model, bias=False)
        self.res_dropout = nn.Dropout(cfg.dropout)
        cos, sin = precompute_freqs_cis(cfg.rope_head_dim, cfg.max_sequence_length, cfg.rope_theta)
        self.register_buffer("freq_cos", cos, persistent=False)
        self.register_buffer("freq_sin", sin, persistent=False)

    def latent_cache(self, x: Tensor) -> tuple[Tensor, Tensor]:
        """What an inference cache needs per token: the normalised kv latent and the rotary key
        (``kv_lora_rank + rope_head_dim`` numbers instead of ``2 * heads * head_dim``)."""
        return self.kv_norm(self.compress_kv(x)), self.k_rope(x)

    def forward(self, x: Tensor) -> Tensor:
        cfg, (b, t, _) = self.cfg, x.shape
        h = cfg.num_heads
        q_latent = self.q_norm(self.compress_q(x))
        q_nope = self.q_nope(q_latent).view(b, t, h, cfg.nope_head_dim)
        q_rope = self.q_rope(q_latent).view(b, t, h, cfg.rope_head_dim)
        kv_latent, k_rope = self.latent_cache(x)
        k_nope = self.k_nope(kv_latent).view(b, t, h, cfg.nope_head_dim)
        v = self.value(kv_latent).view(b, t, h, cfg.v_head_dim)
        q_rope, k_rope = apply_rope(q_rope, k_rope.view(b, t, 1, cfg.rope_head_dim),
                                    (self.freq_cos[:t], self.freq_sin[:t]))
        q = torch.cat([q_nope, q_rope], dim=-1).transpose(1, 2)
        k = torch.cat([k_nope, k_rope.expand(b, t, h, cfg.rope_head_dim)], dim=-1).transpose(1, 2)
        out = F.scaled_dot_product_attention(q, k, v.transpose(1, 2), is_causal=True,
                                             dropout_p=cfg.dropout if self.training else 0.0)
        out = out.transpose(1, 2).reshape(b, t, h * cfg.v_head_dim)
        return self.res_dropout(self.proj(out))
