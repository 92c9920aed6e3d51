"""Print-streaming text generator for any model with ``forward(ids[, kv_cache, position])``
(reference: ohara/inference.py:10-127). For chat use :class:`ohara_b200.chat_engine.ChatEngine`."""

from __future__ import annotations

import time

import torch
import torch.nn as nn


class Inference:
    def __init__(self, model: nn.Module, tokenizer, device: str | torch.device | None = None,
                 temperature: float = 1.0, top_p: float = 0.0, max_new_tokens: int = 500,
                 use_kv_cache: bool = True):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.model = model.to(self.device).eval()
        self.tokenizer = tokenizer
        self.default_temperature = temperature
        self.default_top_p = top_p
        self.max_new_tokens = max_new_tokens
        self.use_kv_cache = use_kv_cache
        self.kv_cache = self._fresh_cache()

    def _fresh_cache(self):
        if self.use_kv_cache and hasattr(self.model, "build_kv_cache"):
            return self.model.build_kv_cache()
        return None

    @staticmethod
    @torch.inference_mode()
    def sampler(logits: torch.Tensor, temperature: float = 1, top_p: float = 0.0) -> torch.Tensor:
        """Greedy when ``temperature <= 0`` or at the defaults (1, 0); otherwise temperature
        sampling, nucleus-restricted for ``0 < top_p < 1`` (the top token always survives)."""
        last = logits[:, -1]
        if temperature <= 0 or (temperature == 1 and top_p <= 0):
            return torch.argmax(last, dim=-1, keepdim=True)
        probs = torch.softmax(last / temperature, dim=-1)
        if top_p <= 0 or top_p >= 1:
            return torch.multinomial(probs, num_samples=1)
        ordered, order = torch.sort(probs, dim=-1, descending=True)
        ordered = ordered.masked_fill(torch.cumsum(ordered, dim=-1) - ordered > top_p, 0.0)
        ordered = ordered / ordered.sum(dim=-1, keepdim=True)
        return torch.gather(order, -1, torch.multinomial(ordered, num_samples=1))

    def generate(self, prompt: str, temperature: float | None = None, top_p: float | None = None,
                 max_new_tokens: int | None = None, stream: bool = True) -> str:
        temperature = self.default_temperature if temperature is None else temperature
        top_p = self.default_top_p if top_p is None else top_p
        max_new_tokens = self.max_new_tokens if max_new_tokens is None else max_new_tokens
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens cannot be negative")
        self.kv_cache = self._fresh_cache()
        token_ids = self.tokenizer.encode(prompt)
        if not token_ids:
            raise ValueError("prompt must encode to at least one token")
        generated = torch.tensor(token_ids, dtype=torch.long, device=self.device).reshape(1, -1)
        limit = getattr(getattr(self.model, "config", None), "max_sequence_length", None)
        if limit is not None:
            if generated.size(1) > limit:
                raise ValueError("prompt exceeds model max_sequence_length")
            max_new_tokens = min(max_new_tokens, max(0, limit - generated.size(1)))
        step_input, position = generated, 0
        started = time.time()
        with torch.inference_mode():
            if stream:
                print(self.tokenizer.decode(generated.tolist()[0]), end="")
            for _ in range(max_new_tokens):
                if self.use_kv_cache:
                    logits = self.model(step_input, self.kv_cache, position)
                else:
                    logits = self.model(generated)
                next_token = self.sampler(logits, temperature=temperature, top_p=top_p)
                if next_token.item() == self.tokenizer.eos_token_id:
                    break
                generated = torch.cat((generated, next_token), dim=-1)
                if self.use_kv_cache:
                    position += step_input.size(1)
                    step_input = next_token
                if stream:
                    print(self.tokenizer.decode([next_token.item()]), end="", flush=True)
        if stream:
            print(f"\nTime: {time.time() - started}s")
        return self.tokenizer.decode(generated.squeeze(0).tolist())
