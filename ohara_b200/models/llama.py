"""Llama-style decoder (dense, loop-MoE or grouped-MoE feed-forwards) — the product model.

Public surface and checkpoint layout follow the reference model (ohara/models/llama.py:16-478):
``Config``, ``Llama.forward(ids[, kv_cache, position_ids]) -> logits``, ``build_kv_cache``,
``num_scaling_params``, ``active_matmul_parameters``, ``estimate_flops`` and state-dict keys
``token_emb, layers.N.attn.{key,query,value,proj}, layers.N.ff.*, layers.N.norm{1,2}, norm,
vocab_proj, freq_cos, freq_sin``.

What is different underneath: every hot op goes through :mod:`ohara_b200.ops`. On a CUDA device in
bf16 autocast the block runs as fused sm_100a kernels in the projection layout ``(B, T, H, D)``
(no head transposes, no KV head expansion for GQA, no mask tensors), activations stay bf16, and
``loss_sum`` fuses the output projection with the cross-entropy so logits are never materialised.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
from torch import Tensor

from ohara_b200 import ops
from ohara_b200.embeddings_pos.rotary import apply_rope, precompute_freqs_cis
from ohara_b200.modules.kv_cache import KVCache
from ohara_b200.modules.mlp import Linear, SwiGLU
from ohara_b200.ops import decode as decode_ops
from ohara_b200.modules.moe import MoE
from ohara_b200.modules.moe_grouped import GroupedMoE
from ohara_b200.modules.norm import RMSNorm


@dataclass
class Config:
    vocab_size: int = 65
    max_sequence_length: int = 64
    hidden_size: int = 128
    intermediate_size: int = 256
    num_attention_heads: int = 4
    num_key_value_heads: int = 0  # 0 = multi-head attention (one KV head per query head)
    num_hidden_layers: int = 4
    dropout: float = 0.2
    multiple_of: int = 4
    bias: bool = False
    weight_tying: bool = False
    rope_theta: float = 100000
    init_style: str = "standard"
    # Mixture of experts: 0 experts keeps every feed-forward dense; with interval N every N-th
    # layer (layer_idx % N == 0) is an MoE.
    moe_num_experts: int = 0
    moe_experts_per_tok: int = 2
    moe_layer_interval: int = 1
    moe_gate_fn: str = "softmax"
    moe_quantile_balancing: bool = True
    moe_grouped: bool = False
    moe_num_shared_experts: int = 0
    moe_normalize_weights: bool = True
    # Extensions over the reference Config (defaults keep its behaviour): Switch-style auxiliary
    # loss coefficient and expert capacity factor for the grouped MoE.
    moe_aux_loss_coef: float = 0.0
    moe_capacity_factor: float | None = None

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads


def validate_config(cfg: Config) -> None:
    if cfg.vocab_size < 2:
        raise ValueError("vocab_size must be at least 2")
    if cfg.hidden_size < 1 or cfg.num_hidden_layers < 1:
        raise ValueError("hidden_size and num_hidden_layers must be positive")
    if cfg.intermediate_size < 1:
        raise ValueError("intermediate_size must be positive")
    if cfg.num_attention_heads < 1 or cfg.hidden_size % cfg.num_attention_heads != 0:
        raise ValueError("hidden_size must be divisible by num_attention_heads")
    if (cfg.hidden_size // cfg.num_attention_heads) % 2 != 0:
        raise ValueError("attention head dimension must be even for rotary embeddings")
    if cfg.max_sequence_length < 2:
        raise ValueError("max_sequence_length must be at least 2")
    kv_heads = cfg.num_key_value_heads or cfg.num_attention_heads
    if kv_heads < 1 or cfg.num_attention_heads % kv_heads != 0:
        raise ValueError("num_key_value_heads must divide num_attention_heads")
    if not 0.0 <= cfg.dropout < 1.0:
        raise ValueError("dropout must be in [0, 1)")
    if cfg.init_style not in {"standard", "nanochat"}:
        raise ValueError("init_style must be 'standard' or 'nanochat'")
    if cfg.init_style == "nanochat" and cfg.weight_tying:
        raise ValueError("nanochat initialization requires untied embeddings")
    if cfg.moe_num_experts < 0 or cfg.moe_num_shared_experts < 0:
        raise ValueError("MoE expert counts cannot be negative")
    if cfg.moe_layer_interval < 1:
        raise ValueError("moe_layer_interval must be positive")
    if cfg.moe_gate_fn not in {"softmax", "sigmoid"}:
        raise ValueError("moe_gate_fn must be 'softmax' or 'sigmoid'")
    if cfg.moe_grouped and cfg.moe_num_experts == 0:
        raise ValueError("moe_grouped requires moe_num_experts > 0")
    if cfg.moe_num_shared_experts > 0 and not cfg.moe_grouped:
        raise ValueError("shared experts require moe_grouped")
    if not cfg.moe_normalize_weights and not cfg.moe_grouped:
        raise ValueError("moe_normalize_weights only applies to grouped MoE")


def _plain_linears(*modules: nn.Module) -> bool:
    """True when every module is an unmodified bias-free ``Linear`` (not a sharded or adapted
    replacement), so that their weights can be handed to a fused op directly."""
    return all(type(m) is Linear and m.bias is None for m in modules)


class Attention(nn.Module):
    def __init__(self, cfg: Config):
        super().__init__()
        d = cfg.hidden_size
        self.num_attention_heads = cfg.num_attention_heads
        self.head_dim = d // cfg.num_attention_heads
        self.num_key_value_heads = cfg.num_key_value_heads or cfg.num_attention_heads
        assert self.num_attention_heads % self.num_key_value_heads == 0
        self.num_queries_per_kv = self.num_attention_heads // self.num_key_value_heads
        self.key = Linear(d, self.head_dim * self.num_key_value_heads, cfg.bias)
        self.query = Linear(d, self.head_dim * self.num_attention_heads, cfg.bias)
        self.value = Linear(d, self.head_dim * self.num_key_value_heads, cfg.bias)
        self.proj = Linear(self.head_dim * self.num_attention_heads, d, cfg.bias)
        self.attn_dropout = nn.Dropout(cfg.dropout)
        self.res_dropout = nn.Dropout(cfg.dropout)
        # Context parallelism: set by ``Llama.enable_context_parallel``. The sequence is then
        # sharded in contiguous chunks over the group and this module exchanges keys / values.
        self.cp_workspace = None

    def forward(self, x: Tensor, mask: Tensor | None, freqs_cis, kv_cache: KVCache | None = None,
                position_ids: int | None = None) -> Tensor:
        batch, seq_len, _ = x.shape
        # Local head counts are derived from the projection widths so a tensor-parallel shard of
        # this module (fewer output features) needs no patching.
        heads = self.query.weight.shape[0] // self.head_dim
        kv_heads = self.key.weight.shape[0] // self.head_dim
        plain = _plain_linears(self.query, self.key, self.value)
        if (plain and kv_cache is None and self.cp_workspace is None and freqs_cis[0] is not None
                and ops.fused_projections(x) and self.head_dim in (64, 128)
                and not (self.training and self.attn_dropout.p > 0.0)):
            # Training / prefill fast path: one q|k|v GEMM; the rotary and attention kernels read
            # their operands as column slices of its output and hand back one gradient for it.
            qkv = ops.linear_cat(x, (self.query.weight, self.key.weight, self.value.weight))
            out = ops.rope_attention(qkv, freqs_cis[0], freqs_cis[1], heads, kv_heads,
                                     self.head_dim)
            return self.res_dropout(self.proj(out.reshape(-1, seq_len, heads * self.head_dim)))
        if (not plain and kv_cache is None and self.cp_workspace is None
                and freqs_cis[0] is not None and self.head_dim in (64, 128)
                and not (self.training and self.attn_dropout.p > 0.0)):
            # The same with the projections sharded over a tensor-parallel group: one gather of
            # the token blocks and one GEMM for this rank's heads of q | k | v.
            from ohara_b200.runtime.tensor_parallel import fused_column_parallel

            qkv = fused_column_parallel(x, (self.query, self.key, self.value))
            if qkv is not None:
                out = ops.rope_attention(qkv, freqs_cis[0], freqs_cis[1], heads, kv_heads,
                                         self.head_dim)
                return self.res_dropout(self.proj(out.reshape(-1, seq_len, heads * self.head_dim)))
        # -1: with sequence-parallel tensor parallelism the projections gather the token blocks of
        # every rank, so they return more sequences than came in.
        if plain:
            q, k, v = ops.linear_fanout(x, (self.query.weight, self.key.weight, self.value.weight))
        else:  # biases, or tensor-parallel replacements of the projections
            q, k, v = self.query(x), self.key(x), self.value(x)
        q = q.view(-1, seq_len, heads, self.head_dim)
        k = k.view(-1, seq_len, kv_heads, self.head_dim)
        v = v.view(-1, seq_len, kv_heads, self.head_dim)
        if (kv_cache is not None and seq_len == 1 and len(freqs_cis) == 4
                and decode_ops.fused_decode_supported(q, kv_cache) and v.dtype == q.dtype):
            # Decode step: RoPE + cache append in one kernel, then attention over the cache in
            # place (no mask tensor, no head expansion, int8 dequantised on the fly).
            q = kv_cache.append_decode(q, k, v, freqs_cis[2], freqs_cis[3], position_ids)
            out = decode_ops.decode_attention(q, kv_cache, position_ids)
            return self.res_dropout(self.proj(out.reshape(-1, 1, heads * self.head_dim)))
        if freqs_cis[0] is None:
            raise ValueError("a device-side position needs the fused decode kernels: bf16 "
                             "activations on CUDA, head_dim 64 or 128, a bf16 or int8 cache")
        q, k = apply_rope(q, k, freqs_cis[:2])
        if self.cp_workspace is not None and kv_cache is None:
            from ohara_b200.parallel.ulysses import UlyssesWorkspace, ulysses_attention

            if isinstance(self.cp_workspace, UlyssesWorkspace):
                # all-to-all mode: whole sequence, this rank's heads, ordinary causal attention
                out = ulysses_attention(q, k.to(q.dtype), v.to(q.dtype), self.cp_workspace,
                                        self.attn_dropout.p, self.training)
                out = out.reshape(-1, seq_len, heads * self.head_dim)
                return self.res_dropout(self.proj(out))
            from ohara_b200.parallel.cp import context_parallel_attention

            bf = torch.bfloat16
            out = context_parallel_attention(q.to(bf), k.to(bf), v.to(bf), self.cp_workspace)
            out = out.reshape(-1, seq_len, heads * self.head_dim)
            return self.res_dropout(self.proj(out))
        if kv_cache is not None:
            assert position_ids is not None
            k, v = kv_cache.forward(k, v.to(k.dtype), position_ids)
        out = ops.attention(
            q, k.to(q.dtype), v.to(q.dtype), causal=True,
            dropout_p=self.attn_dropout.p, training=self.training,
        )
        out = out.reshape(-1, seq_len, heads * self.head_dim)
        return self.res_dropout(self.proj(out))


def uses_moe(cfg: Config, layer_idx: int) -> bool:
    """Whether layer ``layer_idx`` has a mixture-of-experts feed-forward."""
    return cfg.moe_num_experts >= 1 and layer_idx % cfg.moe_layer_interval == 0


class Block(nn.Module):
    def __init__(self, cfg: Config, layer_idx: int = 0):
        super().__init__()
        self.attn = Attention(cfg)
        self.is_moe = uses_moe(cfg, layer_idx)
        if self.is_moe and cfg.moe_grouped:
            self.ff = GroupedMoE(
                dim=cfg.hidden_size, hidden_dim=cfg.intermediate_size,
                num_experts=cfg.moe_num_experts, num_experts_per_tok=cfg.moe_experts_per_tok,
                num_shared_experts=cfg.moe_num_shared_experts, gate_fn=cfg.moe_gate_fn,
                normalize_weights=cfg.moe_normalize_weights,
                quantile_balancing=cfg.moe_quantile_balancing,
                aux_loss_coef=getattr(cfg, "moe_aux_loss_coef", 0.0),
                capacity_factor=getattr(cfg, "moe_capacity_factor", None),
            )
        elif self.is_moe:
            self.ff = MoE(
                dim=cfg.hidden_size, hidden_dim=cfg.intermediate_size,
                num_experts=cfg.moe_num_experts, num_experts_per_tok=cfg.moe_experts_per_tok,
                gate_fn=cfg.moe_gate_fn, quantile_balancing=cfg.moe_quantile_balancing,
            )
        else:
            self.ff = SwiGLU(dim=cfg.hidden_size, hidden_dim=cfg.intermediate_size,
                             dropout=cfg.dropout, bias=cfg.bias)
        self.norm1 = RMSNorm(cfg.hidden_size)
        self.norm2 = RMSNorm(cfg.hidden_size)

    def forward(self, x, mask, freqs_cis, kv_cache: KVCache | None = None,
                position_ids: int | None = None):
        x = x + self.attn(self.norm1(x), mask, freqs_cis, kv_cache, position_ids).to(x.dtype)
        x = x + self.ff(self.norm2(x)).to(x.dtype)
        return x

    def forward_deferred(self, x, pending, freqs_cis, kv_cache: KVCache | None = None,
                         position_ids: int | None = None):
        """Same block, with the residual adds folded into the norms that follow them.

        Takes the residual stream ``x`` plus a branch output ``pending`` that has not been added
        yet (``None`` for the first block) and returns the updated stream and this block's own
        not-yet-added feed-forward output. Mathematically identical to :meth:`forward`; on the
        CUDA fast path each ``add + norm`` pair is one kernel, forward and backward.
        """
        h, x = ops.add_rms_norm(x, pending, self.norm1.weight, self.norm1.eps)
        attn_out = self.attn(h, None, freqs_cis, kv_cache, position_ids)
        h, x = ops.add_rms_norm(x, attn_out, self.norm2.weight, self.norm2.eps)
        return x, self.ff(h)


def _recompute_contexts():
    from contextlib import nullcontext

    from ohara_b200.modules.routing import recomputing

    return nullcontext(), recomputing()


def _checkpointed_block(layer: "Block", h: Tensor, pending: Tensor | None, freqs):
    from torch.utils.checkpoint import checkpoint

    return checkpoint(layer.forward_deferred, h, pending, freqs, use_reentrant=False,
                      context_fn=_recompute_contexts)


class Llama(nn.Module):
    def __init__(self, cfg: Config, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        validate_config(cfg)
        self.config = cfg
        self.token_emb = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([Block(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size)
        self.vocab_proj = Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.weight_tying:
            self.token_emb.weight = self.vocab_proj.weight
        cos, sin = precompute_freqs_cis(cfg.head_dim, cfg.max_sequence_length * 2, cfg.rope_theta)
        self.register_buffer("freq_cos", cos)
        self.register_buffer("freq_sin", sin)
        self.mask = None  # kept for API parity; masks are never materialised here
        # Extension over the reference: recompute every block's activations in the backward pass
        # instead of keeping them (see enable_activation_checkpointing).
        self.activation_checkpointing = False
        self.apply(self._init_weights)
        if cfg.init_style == "nanochat":
            self._init_nanochat_weights()

    # -- forward --------------------------------------------------------------------------------
    def _check_inputs(self, x: Tensor, kv_cache, position_ids) -> int:
        if x.ndim != 2:
            raise ValueError("input token IDs must have shape (batch, sequence)")
        if isinstance(position_ids, Tensor):
            if position_ids.numel() != 1:
                raise ValueError("position_ids must be a scalar cache position")
            position_ids = int(position_ids.item())
        start = 0
        if kv_cache is not None:
            if len(kv_cache) != len(self.layers):
                raise ValueError("KV cache must contain one entry per model layer")
            if position_ids is None or position_ids < 0:
                raise ValueError("a non-negative position_ids is required with KV cache")
            start = position_ids
        elif position_ids is not None:
            raise ValueError("position_ids is only valid when using a KV cache")
        if x.size(1) < 1:
            raise ValueError("input sequence cannot be empty")
        if start + x.size(1) > self.config.max_sequence_length:
            raise ValueError("input exceeds max_sequence_length")
        return start

    def enable_context_parallel(self, workspace, rank: int, world: int) -> None:
        """Shard the sequence over a context-parallel group: this rank then receives its zig-zag
        shard of every sequence (``T / world`` tokens: block ``rank`` and block ``2 * world - 1 -
        rank`` of ``2 * world``, see :func:`ohara_b200.parallel.cp.shard_sequence`), rotary
        positions are the global ones and every attention layer exchanges keys / values through
        ``workspace`` (:class:`ohara_b200.parallel.cp.CPWorkspace` or its lazy form)."""
        self._cp = (rank, world)
        self._cp_positions = None
        for block in self.layers:
            block.attn.cp_workspace = workspace

    def _rope_tables_f32(self) -> tuple[Tensor, Tensor]:
        """Full fp32 rotary tables for the serving kernels (a cached copy when the buffers were
        converted to a lower precision together with the model)."""
        cached = getattr(self, "_rope_f32", None)
        if cached is None or cached[0].device != self.freq_cos.device:
            cached = (self.freq_cos.float().contiguous(), self.freq_sin.float().contiguous())
            self._rope_f32 = cached
        return cached

    def forward_hidden(self, x: Tensor, kv_cache: list[KVCache] | None = None,
                       position_ids: int | Tensor | None = None) -> Tensor:
        """Final-norm hidden states ``(B, T, hidden)`` (everything except the output projection).

        With a KV cache on CUDA, ``position_ids`` may be a one-element int32 CUDA tensor and ``x``
        a single token per sequence: the position is then read on the device by the serving
        kernels and nothing here synchronises with the host, so the step can be captured in a CUDA
        graph (argument checks that would need the value are skipped)."""
        device_position = (
            kv_cache is not None and isinstance(position_ids, Tensor) and position_ids.is_cuda
            and position_ids.dtype == torch.int32 and position_ids.numel() == 1 and x.size(1) == 1
        )
        if kv_cache is not None and getattr(self, "_param_sharding", None) is not None:
            raise NotImplementedError("decoding with a KV cache needs whole parameters: "
                                      "load the full state dict into an unsharded model")
        if device_position:
            h = ops.embedding(x, self.token_emb.weight)
            freqs = (None, None, *self._rope_tables_f32())
            pending = None
            for idx, layer in enumerate(self.layers):
                h, pending = layer.forward_deferred(h, pending, freqs, kv_cache[idx], position_ids)
            return ops.add_rms_norm(h, pending, self.norm.weight, self.norm.eps)[0]
        start = self._check_inputs(x, kv_cache, position_ids)
        seq = x.size(1)
        if getattr(self, "_param_sharding", None) is not None:
            return self._forward_hidden_sharded(x, seq)
        cp = getattr(self, "_cp", None)
        if cp is not None and kv_cache is None:
            if cp[1] * seq > self.config.max_sequence_length:
                raise ValueError("the full sequence exceeds max_sequence_length")
            cached = self._cp_positions
            if cached is None or cached.numel() != seq or cached.device != x.device:
                from ohara_b200.parallel.cp import local_positions

                cached = self._cp_positions = local_positions(cp[0], cp[1], seq, device=x.device)
        h = ops.embedding(x, self.token_emb.weight)
        if cp is not None and kv_cache is None:
            freqs = (self.freq_cos[self._cp_positions], self.freq_sin[self._cp_positions])
        else:
            freqs = (self.freq_cos[start : start + seq], self.freq_sin[start : start + seq])
        if kv_cache is not None and x.is_cuda and seq == 1:
            freqs = (*freqs, *self._rope_tables_f32())
        pending = None
        recompute = (self.activation_checkpointing and kv_cache is None and self.training
                     and torch.is_grad_enabled())
        for idx, layer in enumerate(self.layers):
            if recompute:
                h, pending = _checkpointed_block(layer, h, pending, freqs)
                continue
            cache = kv_cache[idx] if kv_cache is not None else None
            h, pending = layer.forward_deferred(
                h, pending, freqs, cache, start if cache is not None else None
            )
        return ops.add_rms_norm(h, pending, self.norm.weight, self.norm.eps)[0]

    def _forward_hidden_sharded(self, x: Tensor, seq: int) -> Tensor:
        """The same pass with the parameters sharded per block
        (:mod:`ohara_b200.parallel.param_shard`): every unit is gathered just before it runs and
        released after it; the final norm and the output projection stay gathered for the loss
        and the start of the backward pass."""
        sharding = self._param_sharding
        h = sharding.run_unit("embed", lambda ids: ops.embedding(ids, self.token_emb.weight), x)
        cp = getattr(self, "_cp", None)
        if cp is not None:
            if cp[1] * seq > self.config.max_sequence_length:
                raise ValueError("the full sequence exceeds max_sequence_length")
            cached = self._cp_positions
            if cached is None or cached.numel() != seq or cached.device != x.device:
                from ohara_b200.parallel.cp import local_positions

                cached = self._cp_positions = local_positions(cp[0], cp[1], seq, device=x.device)
            freqs = (self.freq_cos[cached], self.freq_sin[cached])
        else:
            freqs = (self.freq_cos[:seq], self.freq_sin[:seq])
        recompute = self.activation_checkpointing and self.training and torch.is_grad_enabled()
        pending = None
        for idx, layer in enumerate(self.layers):
            if recompute:
                block = lambda a, b, layer=layer: _checkpointed_block(layer, a, b, freqs)  # noqa: E731
            else:
                block = lambda a, b, layer=layer: layer.forward_deferred(a, b, freqs)  # noqa: E731
            h, pending = sharding.run_unit(f"layers.{idx}", block, h, pending)
        # (nothing runs after this unit in the forward pass: no gather of a following one)
        sharding.enter_unit("embed" if sharding.tied else "head", prefetch_next=False)
        return ops.add_rms_norm(h, pending, self.norm.weight, self.norm.eps)[0]

    def enable_activation_checkpointing(self, enabled: bool = True) -> "Llama":
        """Keep only each block's input during the forward pass of a training step and run the
        block a second time in the backward pass to rebuild what its gradients need. Activation
        memory drops from everything a block saves (norm outputs, q/k/v, attention output and
        log-sum-exp, gate/up/activation, routed rows) to one residual-stream tensor pair per
        block, for about a third more compute. Routers do not count the recomputed tokens."""
        self.activation_checkpointing = bool(enabled)
        return self

    supports_fused_loss = True

    def forward(self, x: Tensor, kv_cache: list[KVCache] | None = None,
                position_ids: int | Tensor | None = None, *, targets: Tensor | None = None,
                ignore_index: int = -1, loss_scale: Tensor | float | None = None) -> Tensor:
        """Logits ``(B, T, V)``; with ``targets`` the (scaled) summed cross-entropy instead, so a
        wrapper that only forwards ``__call__`` (DDP) can still use the fused loss."""
        if targets is not None:
            return self.loss_sum(x, targets, ignore_index, loss_scale)
        logits = self.vocab_proj(self.forward_hidden(x, kv_cache, position_ids))
        self._release_after_inference()
        return logits

    def _release_after_inference(self) -> None:
        """With sharded parameters and no backward pass to come (evaluation), nothing else would
        release the unit that stays gathered for the loss."""
        sharding = getattr(self, "_param_sharding", None)
        if sharding is not None and not torch.is_grad_enabled():
            sharding.release_all()

    def loss_sum(self, x: Tensor, targets: Tensor, ignore_index: int = -1,
                 scale: Tensor | float | None = None) -> Tensor:
        """``scale * Σ CE(logits, targets)`` over supervised targets, with the output projection
        fused into the loss (no logits tensor). Adds any MoE auxiliary losses (also scaled)."""
        hidden = self.forward_hidden(x)
        if hasattr(self.vocab_proj.weight, "tensor_parallel_dim"):
            raise NotImplementedError("the fused loss needs the whole output projection: a "
                                      "vocabulary-sharded head (mlp_and_head plan) is for inference")
        loss = ops.linear_cross_entropy(hidden, self.vocab_proj.weight, targets, ignore_index, scale)
        aux = self.auxiliary_loss()
        if aux is not None:
            valid = (targets != ignore_index).sum().clamp_min(1).to(loss.dtype)
            aux = aux * valid  # per-token coefficient under a sum-reduced loss
            loss = loss + (aux if scale is None else aux * scale)
        self._release_after_inference()
        return loss

    def auxiliary_loss(self) -> Tensor | None:
        terms = [
            layer.ff.aux_loss
            for layer in self.layers
            if getattr(layer.ff, "aux_loss", None) is not None and self.training
        ]
        return torch.stack(terms).sum() if terms else None

    def build_kv_cache(self, batch_size: int = 1, int8: bool = False) -> list[KVCache]:
        """One empty cache per layer, on the model's device and dtype."""
        if batch_size < 1:
            raise ValueError("batch_size must be at least 1")
        cfg = self.config
        # Local KV heads: a tensor-parallel shard of the model caches only its own heads.
        kv_heads = self.layers[0].attn.key.weight.shape[0] // cfg.head_dim
        shape = (batch_size, cfg.max_sequence_length, kv_heads, cfg.head_dim)
        weight = self.token_emb.weight
        dtype = weight.dtype
        if weight.is_cuda and dtype == torch.float32 and torch.is_autocast_enabled("cuda"):
            dtype = torch.get_autocast_dtype("cuda")
        return [
            KVCache(shape, cfg.max_sequence_length, idx, device=weight.device, dtype=dtype, int8=int8)
            for idx in range(cfg.num_hidden_layers)
        ]

    # -- accounting -----------------------------------------------------------------------------
    def num_scaling_params(self) -> dict[str, int]:
        """Parameter groups used by compute-optimal scaling analysis."""
        token_embeddings = self.token_emb.weight.numel()
        lm_head = 0 if self.vocab_proj.weight is self.token_emb.weight else self.vocab_proj.weight.numel()
        matrices = sum(p.numel() for layer in self.layers for p in layer.parameters() if p.ndim >= 2)
        total = sum(p.numel() for p in self.parameters())
        rest = total - token_embeddings - lm_head - matrices
        if rest < 0:
            raise RuntimeError("parameter groups overlap")
        return {
            "token_embeddings": token_embeddings,
            "lm_head": lm_head,
            "transformer_matrices": matrices,
            "norms_and_scalars": rest,
            "total": total,
            "effective": matrices + lm_head,
        }

    def active_matmul_parameters(self) -> int:
        """Matrix parameters one token passes through (routed experts count k of E)."""
        total = 0
        for block in self.layers:
            total += sum(p.numel() for p in block.attn.parameters() if p.ndim >= 2)
            ff = block.ff
            if isinstance(ff, GroupedMoE):
                per_expert = ff.dim * ff.hidden_dim * 3
                total += per_expert * (ff.num_experts_per_tok + ff.num_shared_experts)
                total += ff.router.weight.numel()
            elif block.is_moe:
                per_expert = sum(p.numel() for p in ff.experts[0].parameters() if p.ndim >= 2)
                total += per_expert * ff.num_experts_per_tok + ff.gate.weight.numel()
            else:
                total += sum(p.numel() for p in ff.parameters() if p.ndim >= 2)
        return total

    def estimate_flops(self, sequence_length: int | None = None) -> float:
        """Forward+backward FLOPs per token: 6·(active matmul params + head) + 12·L·H·D·T."""
        cfg = self.config
        sequence_length = sequence_length or cfg.max_sequence_length
        if not 1 <= sequence_length <= cfg.max_sequence_length:
            raise ValueError("sequence_length must be within the configured context window")
        matmul = self.active_matmul_parameters() + self.vocab_proj.weight.numel()
        attention = 12 * cfg.num_hidden_layers * cfg.num_attention_heads * cfg.head_dim * sequence_length
        return float(6 * matmul + attention)

    # -- init -----------------------------------------------------------------------------------
    def _init_weights(self, module: nn.Module) -> None:
        if isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)
        elif isinstance(module, GroupedMoE):
            for w in (module.w_gate, module.w_up, module.w_down):
                nn.init.normal_(w, mean=0.0, std=0.02)
            module.router_bias.zero_()

    @torch.no_grad()
    def _init_nanochat_weights(self) -> None:
        """Width-transferable init: wide embedding, tiny head, uniform q/k/v and gate/up, zero
        output projections so every block starts as the identity on the residual stream."""
        nn.init.normal_(self.token_emb.weight, mean=0.0, std=0.8)
        nn.init.normal_(self.vocab_proj.weight, mean=0.0, std=0.001)
        bound = math.sqrt(3.0) * self.config.hidden_size**-0.5
        for block in self.layers:
            for proj in (block.attn.query, block.attn.key, block.attn.value):
                nn.init.uniform_(proj.weight, -bound, bound)
            nn.init.zeros_(block.attn.proj.weight)
            if isinstance(block.ff, GroupedMoE):
                block.ff.reset_parameters()
            else:
                experts = block.ff.experts if block.is_moe else [block.ff]
                for expert in experts:
                    nn.init.uniform_(expert.up.weight, -0.4 * bound, 0.4 * bound)
                    nn.init.uniform_(expert.gate.weight, -0.4 * bound, 0.4 * bound)
                    nn.init.zeros_(expert.down.weight)
                if block.is_moe:
                    nn.init.normal_(block.ff.gate.weight, mean=0.0, std=self.config.hidden_size**-0.5)
                    block.ff.router_bias.zero_()
            block.norm1.reset_parameters()
            block.norm2.reset_parameters()
        self.norm.reset_parameters()

    @classmethod
    def from_pretrained(cls, hf_name: str):
        raise NotImplementedError(
            "Llama.from_pretrained is not implemented yet. "
            "Use a model-specific loader or initialize `Llama(Config(...))` directly."
        )
