"""Hawk, Griffin and their multi-query-attention baseline (https://arxiv.org/abs/2402.19427) as
small language models (reference: experiments/griffin_and_hawk/griffin_and_hawk.py:57-364).

The recurrent mixer is :class:`ohara_b200.modules.linear_rnn.Hawk` (causal depth-wise convolution,
real-gated linear recurrent unit on the package's scan, which is a one-pass CUDA kernel on GPUs).
Three block types share the residual layout ``x + mixer(norm(x)); x + GEGLU(norm(x))``:

* ``mqa``: grouped / multi-query attention with rotary positions, optionally a sliding window;
* ``hawk``: the recurrent mixer alone;
* ``griffin``: attention, then the recurrent mixer, then the MLP, each behind its own norm.

Beyond the reference, the recurrent mixer can also be run one token at a time from a constant-size
state (:class:`HawkState`, :func:`hawk_step`), which is what makes these models cheap to decode;
the reference leaves that as a TODO (griffin_and_hawk.py:86).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200.embeddings_pos.rotary import apply_rope, precompute_freqs_cis
from ohara_b200.modules.linear_rnn import Hawk
from ohara_b200.modules.mlp import GEGLU
from ohara_b200.modules.norm import RMSNorm


@dataclass
class HnGConfig:
    model_type: str = "griffin"  # "mqa", "hawk" or "griffin"
    vocab_size: int = 51200
    seq_len: int = 2048
    dim: int = 256
    hidden_dim: int | None = None  # MLP width and recurrent width; default 1.5 * dim
    num_heads: int = 8
    num_kv_heads: int = 1
    num_layers: int = 8
    kernel_size: int = 4
    eps: float = 1e-5
    sliding_window_attention: bool = False
    window_size: int = 128
    weight_tying: bool = True

    @property
    def width(self) -> int:
        return self.hidden_dim or int(self.dim * 1.5)


class GroupedQueryAttention(nn.Module):
    """Causal attention with ``num_kv_heads`` shared key/value heads and an optional local window
    (a query sees itself and the ``window - 1`` positions before it)."""

    def __init__(self, dim: int, num_heads: int, num_kv_heads: int = 1,
                 window: int | None = None) -> None:
        super().__init__()
        if dim % num_heads or num_heads % num_kv_heads:
            raise ValueError("dim must divide into heads and heads into key/value heads")
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.head_dim = dim // num_heads
        self.window = window
        self.query = nn.Linear(dim, dim, bias=False)
        self.key = nn.Linear(dim, self.head_dim * num_kv_heads, bias=False)
        self.value = nn.Linear(dim, self.head_dim * num_kv_heads, bias=False)
        self.proj = nn.Linear(dim, dim, bias=False)

    def forward(self, x: Tensor, freqs: tuple[Tensor, Tensor]) -> Tensor:
        batch, steps, dim = x.shape
        q = self.query(x).view(batch, steps, self.num_heads, self.head_dim)
        k = self.key(x).view(batch, steps, self.num_kv_heads, self.head_dim)
        v = self.value(x).view(batch, steps, self.num_kv_heads, self.head_dim)
        q, k = apply_rope(q, k, freqs)
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        mask = None
        if self.window is not None and self.window < steps:
            distance = torch.arange(steps, device=x.device)[:, None] - torch.arange(steps, device=x.device)
            mask = (distance >= 0) & (distance < self.window)
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=mask is None,
                                             enable_gqa=self.num_kv_heads != self.num_heads)
        return self.proj(out.transpose(1, 2).reshape(batch, steps, dim))


class Block(nn.Module):
    def __init__(self, cfg: HnGConfig) -> None:
        super().__init__()
        kind = cfg.model_type.lower()
        if kind not in ("mqa", "hawk", "griffin"):
            raise ValueError(f"unknown model_type {cfg.model_type!r}")
        window = cfg.window_size if cfg.sliding_window_attention else None
        self.attention = (GroupedQueryAttention(cfg.dim, cfg.num_heads, cfg.num_kv_heads, window)
                          if kind in ("mqa", "griffin") else None)
        self.recurrent = (Hawk(dim=cfg.dim, expansion_factor=cfg.width / cfg.dim,
                               kernel_size=cfg.kernel_size)
                          if kind in ("hawk", "griffin") else None)
        self.mlp = GEGLU(dim=cfg.dim, hidden_dim=cfg.width)
        self.attention_norm = RMSNorm(cfg.dim, eps=cfg.eps) if self.attention is not None else None
        self.recurrent_norm = RMSNorm(cfg.dim, eps=cfg.eps) if self.recurrent is not None else None
        self.mlp_norm = RMSNorm(cfg.dim, eps=cfg.eps)

    def forward(self, x: Tensor, freqs: tuple[Tensor, Tensor]) -> Tensor:
        if self.attention is not None:
            x = x + self.attention(self.attention_norm(x), freqs)
        if self.recurrent is not None:
            x = x + self.recurrent(self.recurrent_norm(x))
        return x + self.mlp(self.mlp_norm(x))


class HawkAndGriffin(nn.Module):
    """Token embedding, ``num_layers`` blocks of one type, layer norm, output projection."""

    def __init__(self, cfg: HnGConfig) -> None:
        super().__init__()
        self.config = cfg
        self.token_emb = nn.Embedding(cfg.vocab_size, cfg.dim)
        self.layers = nn.ModuleList([Block(cfg) for _ in range(cfg.num_layers)])
        self.norm = nn.LayerNorm(cfg.dim)
        self.vocab_proj = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)
        cos, sin = precompute_freqs_cis(cfg.dim // cfg.num_heads, cfg.seq_len * 2)
        self.register_buffer("freq_cos", cos, persistent=False)
        self.register_buffer("freq_sin", sin, persistent=False)
        for module in self.modules():
            if isinstance(module, nn.Embedding):
                nn.init.normal_(module.weight, std=0.02)
        nn.init.normal_(self.vocab_proj.weight, std=0.02)
        if cfg.weight_tying:
            self.token_emb.weight = self.vocab_proj.weight

    def forward(self, tokens: Tensor) -> Tensor:
        steps = tokens.shape[1]
        freqs = (self.freq_cos[:steps], self.freq_sin[:steps])
        x = self.token_emb(tokens)
        for layer in self.layers:
            x = layer(x, freqs)
        return self.vocab_proj(self.norm(x))


# --------------------------------------------------------------------------------------------------
# One token at a time
# --------------------------------------------------------------------------------------------------
@dataclass
class HawkState:
    """What the recurrent mixer carries between tokens: the last ``kernel_size - 1`` inputs of the
    convolution and the hidden state of the linear recurrence (both ``(batch, width)``-sized)."""

    conv_inputs: Tensor  # (batch, kernel_size - 1, width)
    hidden: Tensor       # (batch, width)

    @classmethod
    def zeros(cls, mixer: Hawk, batch: int, device=None, dtype=None) -> "HawkState":
        kernel = mixer.conv.kernel_size[0]
        make = dict(device=device or mixer.output.weight.device,
                    dtype=dtype or mixer.output.weight.dtype)
        return cls(torch.zeros(batch, kernel - 1, mixer.hidden, **make),
                   torch.zeros(batch, mixer.hidden, **make))


def hawk_step(mixer: Hawk, x: Tensor, state: HawkState) -> tuple[Tensor, HawkState]:
    """The mixer's output for ONE new token ``x (batch, dim)`` given ``state``; equals the
    corresponding position of the parallel forward pass over the whole sequence."""
    gate, branch = mixer.proj(x).chunk(2, dim=-1)
    window = torch.cat([state.conv_inputs, branch[:, None]], dim=1)       # (batch, kernel, width)
    # depth-wise causal convolution: weight (width, 1, kernel), newest input last
    mixed = (window * mixer.conv.weight[:, 0].t()).sum(1) + mixer.conv.bias
    rnn = mixer.linear_rnn
    recurrence = rnn.gate_proj(mixed).sigmoid()
    alpha = (-rnn.C * F.softplus(rnn.forget_lambda) * recurrence).exp()
    driven = (1 - alpha**2 + 1e-6).sqrt() * rnn.input_proj(mixed).sigmoid() * mixed
    hidden = alpha * state.hidden + driven
    out = mixer.output(F.gelu(gate) * hidden)
    return out, HawkState(window[:, 1:], hidden)


def parameter_count(cfg: HnGConfig) -> int:
    model = HawkAndGriffin(cfg)
    return sum(p.numel() for p in model.parameters())


def state_floats_per_sequence(cfg: HnGConfig, context: int) -> dict[str, int]:
    """Decode-time memory per sequence, in numbers: the recurrent state is constant, a key/value
    cache grows with the context (or stops at the window)."""
    kind = cfg.model_type.lower()
    recurrent = cfg.num_layers * cfg.width * cfg.kernel_size if kind in ("hawk", "griffin") else 0
    span = min(context, cfg.window_size) if cfg.sliding_window_attention else context
    head_dim = cfg.dim // cfg.num_heads
    cache = cfg.num_layers * 2 * span * cfg.num_kv_heads * head_dim if kind in ("mqa", "griffin") else 0
    return {"recurrent_state": recurrent, "kv_cache": cache}
