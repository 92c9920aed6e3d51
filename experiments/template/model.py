"""The template language model of the experiments: a pre-norm decoder whose attention and
feed-forward layers are pluggable (reference: experiments/template/model.py:20-272 and the copies
of it that every experiment folder carries with one layer swapped).

``TemplateLM(cfg, attention=..., feed_forward=...)`` takes factories ``(cfg) -> nn.Module``; the
attention module is called as ``attention(x, freqs)``, the feed-forward as ``ff(x)`` and may return
``(output, auxiliary_loss)``, in which case the auxiliary terms are averaged into
``model.auxiliary_loss`` (SpringMLP does that). ``VARIANTS`` names the combinations the experiment
folders study; ``build(variant, cfg)`` makes one."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200.embeddings_pos.rotary import precompute_freqs_cis
from ohara_b200.modules.mlp import MLP_MAP
from ohara_b200.modules.norm import RMSNorm


@dataclass
class TemplateConfig:
    vocab_size: int = 256
    seq_len: int = 256
    d_model: int = 128
    hidden_dim: int = 344
    num_heads: int = 4
    num_layers: int = 4
    dropout: float = 0.0
    bias: bool = False
    weight_tying: bool = False
    mlp: str = "swiglu"
    rope_dim: int | None = None   # rotary width; default head_dim


class _Block(nn.Module):
    def __init__(self, cfg: TemplateConfig, attention: Callable, feed_forward: Callable) -> None:
        super().__init__()
        self.attn, self.ff = attention(cfg), feed_forward(cfg)
        self.norm1, self.norm2 = RMSNorm(cfg.d_model), RMSNorm(cfg.d_model)

    def forward(self, x: Tensor, freqs) -> tuple[Tensor, Tensor | None]:
        x = x + self.attn(self.norm1(x), freqs)
        out = self.ff(self.norm2(x))
        out, aux = out if isinstance(out, tuple) else (out, None)
        # a layer that iterates on its input (SpringMLP) returns the updated state itself
        return (out if getattr(self.ff, "includes_residual", False) else x + out), aux


class TemplateLM(nn.Module):
    def __init__(self, cfg: TemplateConfig, attention: Callable | None = None,
                 feed_forward: Callable | None = None) -> None:
        super().__init__()
        from experiments.partial_kv.pkv import FullAttention

        attention = attention or (lambda c: FullAttention(c.d_model, c.num_heads, c.dropout, c.bias))
        feed_forward = feed_forward or (lambda c: MLP_MAP[c.mlp](c.d_model, c.hidden_dim))
        self.config = cfg
        self.token_emb = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(_Block(cfg, attention, feed_forward) for _ in range(cfg.num_layers))
        self.norm = RMSNorm(cfg.d_model)
        self.vocab_proj = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.weight_tying:
            self.token_emb.weight = self.vocab_proj.weight
        cos, sin = precompute_freqs_cis(cfg.rope_dim or cfg.d_model // cfg.num_heads, cfg.seq_len)
        self.register_buffer("freq_cos", cos, persistent=False)
        self.register_buffer("freq_sin", sin, persistent=False)
        self.auxiliary_loss: Tensor | None = None

    def forward(self, tokens: Tensor) -> Tensor:
        steps = tokens.shape[1]
        freqs = (self.freq_cos[:steps], self.freq_sin[:steps])
        x = self.token_emb(tokens)
        extras = []
        for layer in self.layers:
            x, aux = layer(x, freqs)
            if aux is not None:
                extras.append(aux.mean())
        self.auxiliary_loss = torch.stack(extras).mean() if extras else None
        return self.vocab_proj(self.norm(x))


def _variants() -> dict[str, Callable[[TemplateConfig], TemplateLM]]:
    from experiments.deglu.deglu import DeGLU
    from experiments.partial_kv.pkv import KeyValueTiedAttention, PartialKVAttention
    from experiments.springnet.springnet import SpringMLP
    from experiments.xglu.xglu import XGLU

    from experiments.misc.small_modules import Pattention, XLinear, relu_squared
    from experiments.mixture_of_depth.mod import MixtureOfDepth
    from experiments.template.monkey_patcher import patch_linears

    class ReLUSquaredMLP(nn.Module):
        def __init__(self, dim: int, hidden: int) -> None:
            super().__init__()
            self.up, self.down = nn.Linear(dim, hidden, bias=False), nn.Linear(hidden, dim, bias=False)

        def forward(self, x: Tensor) -> Tensor:
            return self.down(relu_squared(self.up(x)))

    class DepthRoutedMLP(nn.Module):
        """Half of the tokens of a sequence go through the MLP, chosen by a router; in training
        the auxiliary router that decoding relies on is fitted alongside."""

        includes_residual = True

        def __init__(self, dim: int, hidden: int) -> None:
            super().__init__()
            self.routed = MixtureOfDepth(MLP_MAP["swiglu"](dim, hidden), dim, capacity_factor=0.5)

        def forward(self, x: Tensor):
            out, aux = self.routed(x, auxiliary_loss=self.training)
            return out if aux is None else (out, aux)

    class LatentAttention(nn.Module):
        """Multi-head latent attention (it carries its own rotary tables) behind the template's
        ``attention(x, freqs)`` interface."""

        def __init__(self, cfg: TemplateConfig) -> None:
            super().__init__()
            from experiments.mla.mla import MLAConfig, MultiHeadLatentAttention

            head = cfg.d_model // cfg.num_heads
            self.inner = MultiHeadLatentAttention(MLAConfig(
                d_model=cfg.d_model, num_heads=cfg.num_heads, v_head_dim=head,
                nope_head_dim=head // 2, rope_head_dim=head // 2, q_lora_rank=cfg.d_model // 2,
                kv_lora_rank=cfg.d_model // 4, max_sequence_length=cfg.seq_len))

        def forward(self, x: Tensor, freqs) -> Tensor:
            return self.inner(x)

    class ParameterTokenAttention(nn.Module):
        """Attention whose four projections are parameter-token attention layers, so that the
        whole block is made of attention over learned tokens (the Tokenformer block)."""

        def __init__(self, cfg: TemplateConfig) -> None:
            super().__init__()
            from experiments.partial_kv.pkv import _attend, _heads
            from ohara_b200.embeddings_pos.rotary import apply_rope

            self._attend, self._heads, self._rope = _attend, _heads, apply_rope
            self.num_heads = cfg.num_heads
            tokens = cfg.d_model
            self.query, self.key, self.value, self.proj = (
                Pattention(cfg.d_model, cfg.d_model, tokens) for _ in range(4))

        def forward(self, x: Tensor, freqs) -> Tensor:
            q, k = self._rope(self._heads(self.query(x), self.num_heads),
                              self._heads(self.key(x), self.num_heads), freqs)
            v = self._heads(self.value(x), self.num_heads)
            return self.proj(self._attend(q, k, v, 0.0, self.training))

    def hypersphere(cfg: TemplateConfig) -> TemplateLM:
        model = TemplateLM(cfg)

        def to_xlinear(linear: nn.Linear) -> XLinear:
            new = XLinear(linear.in_features, linear.out_features, linear.bias is not None)
            new.load_state_dict(linear.state_dict())
            return new

        for layer in model.layers:  # the blocks' projections; embedding and head stay plain
            patch_linears(layer, build=to_xlinear)
        return model

    def bitnet(cfg: TemplateConfig) -> TemplateLM:
        from experiments.bitnet.bitnet import apply_bitlinear

        model = TemplateLM(cfg)
        for layer in model.layers:  # 1.58-bit projections in the blocks; embedding and head stay plain
            apply_bitlinear(layer)
        return model

    def with_rope(cfg: TemplateConfig, width: int) -> TemplateConfig:
        return TemplateConfig(**{**cfg.__dict__, "rope_dim": width})

    return {
        "baseline": lambda c: TemplateLM(c),
        "kattention": lambda c: TemplateLM(
            c, attention=lambda k: KeyValueTiedAttention(k.d_model, k.num_heads, k.dropout, k.bias)),
        "partial_kv": lambda c: TemplateLM(
            with_rope(c, c.d_model // c.num_heads // 2),
            attention=lambda k: PartialKVAttention(k.d_model, k.num_heads, k.dropout, k.bias)),
        "xglu": lambda c: TemplateLM(
            c, feed_forward=lambda k: XGLU(k.d_model, k.hidden_dim, xglu_rank=max(8, k.d_model // 8))),
        "deglu": lambda c: TemplateLM(c, feed_forward=lambda k: DeGLU(k.d_model, k.hidden_dim - k.hidden_dim % 4)),
        "springnet": lambda c: TemplateLM(
            c, feed_forward=lambda k: SpringMLP(k.d_model, k.hidden_dim, spring_steps=4)),
        "tokenformer": lambda c: TemplateLM(
            c, feed_forward=lambda k: Pattention(k.d_model, k.d_model, num_tokens=k.hidden_dim)),
        "tokenformer_full": lambda c: TemplateLM(
            c, attention=ParameterTokenAttention,
            feed_forward=lambda k: Pattention(k.d_model, k.d_model, num_tokens=k.hidden_dim)),
        "mla": lambda c: TemplateLM(c, attention=LatentAttention),
        "relu2": lambda c: TemplateLM(c, feed_forward=lambda k: ReLUSquaredMLP(k.d_model, k.hidden_dim)),
        "mixture_of_depth": lambda c: TemplateLM(
            c, feed_forward=lambda k: DepthRoutedMLP(k.d_model, k.hidden_dim)),
        "hypersphere": hypersphere,
        "bitnet": bitnet,
    }


VARIANTS = tuple(_variants())


def build(variant: str, cfg: TemplateConfig) -> TemplateLM:
    return _variants()[variant](cfg)
