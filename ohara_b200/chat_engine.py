"""Streaming chat inference over a finetuned checkpoint.

``ChatEngine`` couples a :class:`Llama` with a chat tokenizer and yields decoded text deltas while
it samples (text is emitted by diffing the decode of the whole reply, which is BPE-safe). The
checkpoint carries only a state dict, so the architecture is recovered from tensor shapes by
:func:`config_from_state_dict`. Reference behaviour: ohara/chat_engine.py:33-422.

Additions for serving on a B200: ``generate_batch`` decodes a whole batch of prompts with one KV
cache and no per-token host synchronisation (the sampled token stays on the device), which is what
the batch-1/16/64 decode benchmark drives.
"""

from __future__ import annotations

import json
from collections.abc import Iterator, Mapping, Sequence
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch

from ohara_b200.chat import (
    ASSISTANT_END,
    load_chat_tokenizer,
    render_for_completion,
    special_token_ids,
)
from ohara_b200.models.llama import Config, Llama


@dataclass
class SamplingConfig:
    temperature: float = 0.8
    top_p: float = 0.95
    top_k: int = 0
    max_new_tokens: int = 512

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature cannot be negative")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must be in [0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k cannot be negative")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")


def sample_next_token(logits: torch.Tensor, config: SamplingConfig,
                      generator: torch.Generator | None = None) -> torch.Tensor:
    """Sample ``(batch, 1)`` token ids from the last position of ``logits (batch, seq, vocab)``.

    Order: temperature (0 = greedy argmax) → top-k threshold → softmax → top-p, where a token is
    dropped when the mass *before* it already exceeds ``top_p`` (so the most likely token always
    survives) → renormalise → multinomial.
    """
    if logits.is_cuda:
        # One fused kernel per step (mask, top-k, softmax, top-p, draw) instead of sort + cumsum +
        # multinomial; the draw uses one uniform number per row from `generator`.
        from ohara_b200.ops.decode import sample

        last = logits[:, -1]
        uniforms = None
        if config.temperature > 0:
            uniforms = torch.rand(last.size(0), device=last.device, dtype=torch.float32,
                                  generator=generator)
        return sample(last, temperature=config.temperature, top_k=config.top_k,
                      top_p=config.top_p, uniforms=uniforms)
    last = logits[:, -1].float()
    if config.temperature == 0:
        return last.argmax(dim=-1, keepdim=True)
    last = last / config.temperature
    if config.top_k > 0:
        k = min(config.top_k, last.size(-1))
        kth = last.topk(k, dim=-1).values[:, -1:]
        last = last.masked_fill(last < kth, float("-inf"))
    probs = torch.softmax(last, dim=-1)
    if 0.0 < config.top_p < 1.0:
        ordered, order = torch.sort(probs, dim=-1, descending=True)
        mass_before = torch.cumsum(ordered, dim=-1) - ordered
        ordered = ordered.masked_fill(mass_before > config.top_p, 0.0)
        ordered = ordered / ordered.sum(dim=-1, keepdim=True)
        pick = torch.multinomial(ordered, num_samples=1, generator=generator)
        return torch.gather(order, -1, pick)
    return torch.multinomial(probs, num_samples=1, generator=generator)


_WRAPPER_PREFIXES = ("module.", "_orig_mod.")


def strip_wrapper_prefixes(key: str) -> str:
    """Remove any leading ``module.`` (DDP) / ``_orig_mod.`` (torch.compile) prefixes, in any
    order and any number."""
    stripped = True
    while stripped:
        stripped = False
        for prefix in _WRAPPER_PREFIXES:
            if key.startswith(prefix):
                key = key[len(prefix):]
                stripped = True
    return key


def _clean_state_dict(state: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    return {strip_wrapper_prefixes(key): value for key, value in state.items()}


def _layers_with(state: Mapping[str, torch.Tensor], predicate) -> list[int]:
    return sorted({int(k.split(".")[1]) for k in state if k.startswith("layers.") and predicate(k)})


def config_from_state_dict(state: Mapping[str, torch.Tensor], *, moe_experts_per_tok: int = 2,
                           moe_gate_fn: str = "softmax",
                           moe_normalize_weights: bool = True) -> Config:
    """Rebuild a :class:`Config` from checkpoint tensor shapes.

    Shapes determine everything except the routing choices (top-k, gate function, sigmoid
    normalisation), which the caller supplies. Head dimension and context length come from the
    rotary table, stored at twice the context: ``freq_cos (2·T, D/2)``.
    """
    freq_cos = state.get("freq_cos")
    if freq_cos is None:
        raise ValueError("checkpoint has no rotary buffer; cannot infer head dimension")
    head_dim = int(freq_cos.shape[-1]) * 2
    context = int(freq_cos.shape[0]) // 2
    vocab_size, hidden_size = (int(v) for v in state["token_emb.weight"].shape)
    num_layers = 1 + max(int(k.split(".")[1]) for k in state if k.startswith("layers."))
    heads = int(state["layers.0.attn.query.weight"].shape[0]) // head_dim
    kv_heads = int(state["layers.0.attn.key.weight"].shape[0]) // head_dim
    common = dict(
        vocab_size=vocab_size, hidden_size=hidden_size, max_sequence_length=context,
        num_hidden_layers=num_layers, num_attention_heads=heads,
        num_key_value_heads=0 if kv_heads == heads else kv_heads, dropout=0.0,
        weight_tying=state["vocab_proj.weight"].data_ptr() == state["token_emb.weight"].data_ptr(),
    )

    def interval(layers: list[int]) -> int:
        return layers[1] - layers[0] if len(layers) > 1 else num_layers

    grouped = _layers_with(state, lambda k: k.endswith(".ff.w_gate"))
    if grouped:
        first = grouped[0]
        experts, _, width = (int(v) for v in state[f"layers.{first}.ff.w_gate"].shape)
        shared = state.get(f"layers.{first}.ff.shared_gate.weight")
        return Config(
            **common, intermediate_size=width, moe_num_experts=experts,
            moe_experts_per_tok=moe_experts_per_tok, moe_layer_interval=interval(grouped),
            moe_grouped=True,
            moe_num_shared_experts=int(shared.shape[0]) // width if shared is not None else 0,
            moe_gate_fn=moe_gate_fn, moe_normalize_weights=moe_normalize_weights,
        )
    looped = _layers_with(state, lambda k: ".ff.experts." in k)
    if looped:
        first = looped[0]
        experts = 1 + max(int(k.split(".")[4]) for k in state
                          if k.startswith(f"layers.{first}.ff.experts."))
        width = int(state[f"layers.{first}.ff.experts.0.up.weight"].shape[0])
        return Config(**common, intermediate_size=width, moe_num_experts=experts,
                      moe_experts_per_tok=moe_experts_per_tok, moe_layer_interval=interval(looped),
                      moe_gate_fn=moe_gate_fn)
    return Config(**common, intermediate_size=int(state["layers.0.ff.up.weight"].shape[0]))


class ChatEngine:
    def __init__(self, model: Llama, tokenizer, *, device: str | torch.device | None = None,
                 dtype: torch.dtype | None = None) -> None:
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.model = model.to(device=self.device, dtype=self.dtype).eval()
        self.tokenizer = tokenizer
        self.specials = special_token_ids(tokenizer)
        self.assistant_end_id = self.specials[ASSISTANT_END]
        self.eos_token_id = tokenizer.eos_token_id
        # Rows at or above the tokenizer size only pad the matmul; they must never be sampled.
        self.tokenizer_vocab_size = len(tokenizer)
        self.max_sequence_length = model.config.max_sequence_length

    @classmethod
    def from_checkpoint(cls, checkpoint_path: str | Path, *,
                        tokenizer_dir: str | Path | None = None,
                        tokenizer_name: str = "EleutherAI/gpt-neo-125m",
                        device: str | torch.device | None = None,
                        dtype: torch.dtype | None = None, moe_experts_per_tok: int = 2,
                        moe_gate_fn: str = "softmax",
                        moe_normalize_weights: bool = True) -> "ChatEngine":
        """Load a ``.pt`` written by the trainers. A tokenizer directory saved beside the
        checkpoint (``sft.pt`` → ``sft/``) is preferred over ``tokenizer_name``."""
        checkpoint_path = Path(checkpoint_path)
        if not checkpoint_path.exists():
            raise FileNotFoundError(f"checkpoint not found: {checkpoint_path}")
        if tokenizer_dir is None:
            beside = checkpoint_path.with_suffix("")
            tokenizer_dir = beside if (beside / "tokenizer.json").exists() else None
        if tokenizer_dir is not None:
            tokenizer = load_chat_tokenizer(tokenizer_dir=tokenizer_dir, prefer_hf=False,
                                            local_files_only=True)
        else:
            tokenizer = load_chat_tokenizer(hf_name=tokenizer_name)
        checkpoint = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
        state = _clean_state_dict(checkpoint.get("model", checkpoint))
        config = config_from_state_dict(
            state, moe_experts_per_tok=moe_experts_per_tok, moe_gate_fn=moe_gate_fn,
            moe_normalize_weights=moe_normalize_weights,
        )
        if config.vocab_size < len(tokenizer):
            raise ValueError(
                f"checkpoint vocabulary ({config.vocab_size:,}) is smaller than the tokenizer "
                f"({len(tokenizer):,}). Point --tokenizer-dir at the directory saved next to the "
                "checkpoint."
            )
        model = Llama(config)
        model.load_state_dict(state, strict=True)
        return cls(model, tokenizer, device=device, dtype=dtype)

    def metadata(self, checkpoint_path: str | Path | None = None) -> dict[str, Any]:
        cfg = self.model.config
        info: dict[str, Any] = {
            "parameters": sum(p.numel() for p in self.model.parameters()),
            "layers": cfg.num_hidden_layers,
            "hidden_size": cfg.hidden_size,
            "heads": cfg.num_attention_heads,
            "context_length": self.max_sequence_length,
            "vocab_size": cfg.vocab_size,
            "device": str(self.device),
            "dtype": str(self.dtype).removeprefix("torch."),
        }
        if checkpoint_path is not None:
            sidecar = Path(checkpoint_path).with_suffix("") / "ohara_chat.json"
            if sidecar.exists():
                try:
                    info["sft"] = json.loads(sidecar.read_text(encoding="utf-8"))
                except json.JSONDecodeError:
                    pass
        return info

    def render_prompt(self, messages: Sequence[Mapping[str, Any]]) -> list[int]:
        """Prompt ids that leave room for a reply: whole leading turns are dropped until it fits."""
        budget = self.max_sequence_length
        turns = list(messages)
        while turns:
            ids = render_for_completion(self.tokenizer, turns, max_tokens=budget)
            if len(ids) < budget:
                return ids
            turns = turns[2:] if len(turns) > 2 else turns[1:]
        raise ValueError("the latest message alone does not fit in the context window")

    def _mask_padding_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        if logits.size(-1) > self.tokenizer_vocab_size:
            logits[..., self.tokenizer_vocab_size:] = float("-inf")
        return logits

    @torch.inference_mode()
    def generate_stream(self, messages: Sequence[Mapping[str, Any]],
                        config: SamplingConfig | None = None, *,
                        seed: int | None = None) -> Iterator[str]:
        """Yield text deltas of the assistant's reply until ``<|assistant_end|>``, EOS, or the
        token / context budget runs out."""
        config = config or SamplingConfig()
        prompt = self.render_prompt(messages)
        room = self.max_sequence_length - len(prompt)
        if room < 1:
            raise ValueError("no room left in the context window for a reply")
        generator = None
        if seed is not None:
            generator = torch.Generator(device=self.device).manual_seed(seed)
        cache = self.model.build_kv_cache(batch_size=1)
        step_input = torch.tensor(prompt, dtype=torch.long, device=self.device).view(1, -1)
        position = 0
        produced: list[int] = []
        emitted = ""
        for _ in range(min(config.max_new_tokens, room)):
            logits = self._mask_padding_vocab(self.model(step_input, cache, position))
            position += step_input.size(1)
            next_token = sample_next_token(logits, config, generator)
            token_id = int(next_token.item())
            if token_id == self.assistant_end_id or token_id == self.eos_token_id:
                break
            produced.append(token_id)
            step_input = next_token
            text = self.tokenizer.decode(produced, skip_special_tokens=True)
            if len(text) > len(emitted):
                yield text[len(emitted):]
                emitted = text

    def generate(self, messages: Sequence[Mapping[str, Any]], config: SamplingConfig | None = None,
                 *, seed: int | None = None) -> str:
        return "".join(self.generate_stream(messages, config, seed=seed))

    @torch.inference_mode()
    def generate_batch(self, prompt_ids: torch.Tensor, config: SamplingConfig | None = None, *,
                       seed: int | None = None, stop_on_end: bool = False,
                       cuda_graph: bool = True) -> torch.Tensor:
        """Decode ``max_new_tokens`` tokens for a ``(batch, prompt_len)`` tensor of prompts of
        equal length. Returns ``(batch, new_tokens)`` ids.

        On CUDA (bf16 model, no early stop) the prompt is prefilled once and every further step —
        model forward, sampling, writing the token back as the next input, advancing the position —
        runs without the host: positions and the step counter live on the device and the step is
        replayed from a CUDA graph (``cuda_graph=False`` issues the same kernels eagerly). Otherwise
        a plain loop is used; it copies to the host only when ``stop_on_end`` asks for an early exit
        once every row has finished."""
        config = config or SamplingConfig()
        prompt_ids = prompt_ids.to(self.device)
        batch, prompt_len = prompt_ids.shape
        room = self.max_sequence_length - prompt_len
        if room < 1:
            raise ValueError("no room left in the context window for a reply")
        steps = min(config.max_new_tokens, room)
        generator = None
        if seed is not None:
            generator = torch.Generator(device=self.device).manual_seed(seed)
        cache = self.model.build_kv_cache(batch_size=batch)
        if self._device_loop_supported() and not stop_on_end:
            return self._generate_on_device(prompt_ids, cache, config, steps, generator, cuda_graph)
        out = torch.empty(batch, steps, dtype=torch.long, device=self.device)
        finished = torch.zeros(batch, dtype=torch.bool, device=self.device)
        step_input, position = prompt_ids, 0
        for step in range(steps):
            logits = self._mask_padding_vocab(self.model(step_input, cache, position))
            position += step_input.size(1)
            step_input = sample_next_token(logits, config, generator)
            out[:, step] = step_input[:, 0]
            if stop_on_end:
                finished |= (step_input[:, 0] == self.assistant_end_id)
                if self.eos_token_id is not None:
                    finished |= step_input[:, 0] == self.eos_token_id
                if bool(finished.all()):
                    return out[:, : step + 1]
        return out

    def _device_loop_supported(self) -> bool:
        cfg = self.model.config
        return (self.device.type == "cuda" and self.dtype == torch.bfloat16
                and cfg.head_dim in (64, 128)
                and cfg.num_attention_heads // cfg.kv_heads in (1, 2, 4, 8))

    def _generate_on_device(self, prompt_ids, cache, config: SamplingConfig, steps: int,
                            generator, cuda_graph: bool) -> torch.Tensor:
        from ohara_b200.ops.decode import sample

        batch, prompt_len = prompt_ids.shape
        device = self.device
        out = torch.empty(batch, steps, dtype=torch.long, device=device)
        token = torch.empty(batch, 1, dtype=torch.long, device=device)
        # [step, position of the token about to be fed, rows finished in the current step]
        counters = torch.tensor([0, prompt_len - 1, 0], dtype=torch.int32, device=device)
        position = counters[1:2]
        uniforms = None
        if config.temperature > 0:
            uniforms = torch.rand(steps, batch, device=device, dtype=torch.float32,
                                  generator=generator)
        draw = dict(temperature=config.temperature, top_k=config.top_k, top_p=config.top_p,
                    valid_vocab=self.tokenizer_vocab_size, uniforms=uniforms, out=out,
                    next_input=token.view(-1), counters=counters)

        logits = self.model(prompt_ids, cache, 0)
        sample(logits[:, -1], **draw)  # writes column 0; position becomes prompt_len

        def step() -> None:
            step_logits = self.model(token, cache, position)
            sample(step_logits[:, -1], **draw)

        remaining = steps - 1
        if remaining > 0 and cuda_graph and remaining > 2:
            step()  # eager warm-up: lazy initialisation must not happen during capture
            remaining -= 1
            graph = torch.cuda.CUDAGraph()
            try:
                # thread_local: helper threads of a process group (tensor-parallel decoding) may
                # query events while this thread captures.
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    step()
            except RuntimeError:
                graph = None  # something in the step cannot be captured: fall back to eager
            if graph is not None:
                remaining -= 1  # capture does not run the step; the first replay does
                graph.replay()
                for _ in range(remaining):
                    graph.replay()
                remaining = 0
        for _ in range(remaining):
            step()
        for layer_cache in cache:
            layer_cache.set_length(prompt_len + steps - 1, batch)
        return out
