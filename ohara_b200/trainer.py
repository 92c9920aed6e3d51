"""Training loop.

Behavioural contract of the reference trainer (ohara/trainer.py:44-584) is kept: 1-based
iterations, ``lr * lr_scale`` per group, momentum / weight-decay schedules applied to Muon groups
only, loss = Σ cross-entropy over all micro-batches ÷ number of supervised targets of the step,
non-finite guards, the ``iter | loss | lr | time | tok/s | mfu | eta`` line, fp64 evaluation
accumulators with bits-per-byte, cached validation batches, and the checkpoint keys.

Differences that matter on a B200: when the model advertises ``supports_fused_loss`` the step
calls ``model(data, targets=..., loss_scale=1/valid)`` so the output projection and the
cross-entropy run as one chunked kernel sequence and no logits tensor exists; the valid-token
count stays on the device (no per-step ``.item()`` before the forward); step time is measured
with CUDA events; and the MFU denominator knows the B200.
"""

from __future__ import annotations

import gc
import json
import math
import os
import time
from collections import deque
from collections.abc import Callable, Mapping
from contextlib import nullcontext
from pathlib import Path
from typing import Any, Protocol

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
import torch.optim as optim
from torch.utils.data import DataLoader

from ohara_b200.utils.profiling import DeviceTimer, nvtx_range
from ohara_b200.utils.tools import BetterCycle


class RuntimeEngine(Protocol):
    device: torch.device
    is_global_zero: bool
    data_parallel_world_size: int

    def launch(self) -> None: ...
    def prepare_dataloaders(self, *dataloaders: DataLoader): ...
    def prepare(self, module: nn.Module, *optimizers: optim.Optimizer): ...
    def prepare_optimizers(self, *optimizers: optim.Optimizer): ...
    def to_device(self, value: Any) -> Any: ...
    def autocast_context(self): ...
    def no_backward_sync(self, module: nn.Module, enabled: bool = True): ...
    def backward(self, loss: torch.Tensor) -> None: ...
    def clip_gradients(self, model: nn.Module, optimizer: optim.Optimizer, max_norm: float) -> torch.Tensor: ...
    def optimizer_step(self, optimizer: optim.Optimizer) -> None: ...
    def synchronize(self) -> None: ...
    def save(self, path: str | Path, state: dict[str, Any]) -> None: ...
    def log_dict(self, payload: dict[str, Any], step: int | None = None) -> None: ...


# Dense bf16 tensor-core peaks (FLOP/s) by device-name substring. The B200 entry is the nominal
# dense figure; a measured sustained value, when the host provides one, takes precedence
# (see `measured_peak_flops`).
PEAK_BF16_FLOPS = {
    "B200": 2.25e15,
    "GB200": 2.25e15,
    "B100": 1.8e15,
    "H100": 9.89e14,
    "H200": 9.89e14,
    "A100": 3.12e14,
    "A800": 3.12e14,
    "L40S": 3.62e14,
    "L40": 1.81e14,
    "RTX 4090": 1.65e14,
    "RTX 6000 ADA": 1.46e14,
}


def measured_peak_flops(search_from: Path | None = None) -> float | None:
    """Sustained bf16 matmul FLOP/s from a ``MEASURED_PEAKS.json`` next to the package root or
    named by ``OHARA_MEASURED_PEAKS``; ``None`` if there is no such file."""
    candidates = []
    if os.environ.get("OHARA_MEASURED_PEAKS"):
        candidates.append(Path(os.environ["OHARA_MEASURED_PEAKS"]))
    root = (search_from or Path(__file__)).resolve().parent.parent
    candidates.append(root / "MEASURED_PEAKS.json")
    for path in candidates:
        try:
            data = json.loads(path.read_text())
            value = data.get("bf16_tflops_sustained") or data.get("bf16_tflops")
            if value:
                return float(value) * 1e12
        except (OSError, ValueError):
            continue
    return None


def _unwrap(model: nn.Module) -> nn.Module:
    return model.module if hasattr(model, "module") and isinstance(model.module, nn.Module) else model


class Trainer:
    def __init__(
        self,
        engine: RuntimeEngine,
        model: nn.Module,
        optimizer: optim.Optimizer,
        train_dataloader: DataLoader,
        val_dataloader: DataLoader,
        get_lr: Callable[[int], float],
        micro_batch: int,
        max_iters: int,
        eval_iters: int,
        save_ckpt_iters: int,
        get_optimizer_hparams: Callable[[int], Mapping[str, float]] | None = None,
        ignore_index: int = -1,
        push_to_hub: bool = False,
        model_name: str = "",
        log_iter_loss: bool = False,
        iter_loss_window: int = 100,
        print_every: int = 1,
        eval_val_batches: int = 100,
        eval_train_batches: int = 0,
        grad_clip_norm: float | None = None,
        flops_per_token: float | None = None,
        peak_flops: float | None = None,
        timing_warmup_steps: int = 10,
        cudagraph_mark_step_begin: bool = False,
        checkpoint_path: str | Path = "./ckpt/model.pt",
        token_bytes: torch.Tensor | None = None,
        apply_router_balancing: Callable[[nn.Module], None] | None = None,
        fused_loss: bool | None = None,
        profile_sections: bool = False,
    ):
        if micro_batch < 1:
            raise ValueError("micro_batch must be at least 1")
        if max_iters < 1:
            raise ValueError("max_iters must be at least 1")
        if eval_iters < 0 or save_ckpt_iters < 0:
            raise ValueError("eval_iters and save_ckpt_iters cannot be negative")
        if eval_val_batches < 1:
            raise ValueError("eval_val_batches must be at least 1")
        if iter_loss_window < 1:
            raise ValueError("iter_loss_window must be at least 1")
        if token_bytes is not None and token_bytes.ndim != 1:
            raise ValueError("token_bytes must be a one-dimensional vocabulary lookup")
        self.engine = engine
        self.model = model
        self.optimizer = optimizer
        self.train_dataloader = BetterCycle(train_dataloader)
        self.val_dataloader = BetterCycle(val_dataloader)
        self.get_lr = get_lr
        self.get_optimizer_hparams = get_optimizer_hparams
        self.micro_batch = micro_batch
        self.max_iters = max_iters
        self.eval_iters = eval_iters
        self.save_ckpt_iters = save_ckpt_iters
        self.ignore_index = ignore_index
        self.push_to_hub = push_to_hub
        self.model_name = model_name
        self.log_iter_loss = log_iter_loss
        self.iter_loss_window = iter_loss_window
        self.print_every = max(1, int(print_every))
        self.eval_val_batches = max(1, int(eval_val_batches))
        self.eval_train_batches = max(0, int(eval_train_batches))
        self.grad_clip_norm = grad_clip_norm
        self.flops_per_token = flops_per_token
        self.peak_flops = peak_flops
        self.timing_warmup_steps = max(0, int(timing_warmup_steps))
        self.cudagraph_mark_step_begin = cudagraph_mark_step_begin
        self.checkpoint_path = Path(checkpoint_path)
        self.apply_router_balancing = apply_router_balancing
        # Device time per phase of the step (CUDA events, max over ranks in ``section_times``);
        # without it the phases are still NVTX ranges when those are switched on.
        self.timer: DeviceTimer | None = None
        if profile_sections:
            self.timer = DeviceTimer(getattr(engine, "device", None))
        self.token_bytes = self.engine.to_device(token_bytes) if token_bytes is not None else None
        self.iter_loss_history: deque[float] = deque(maxlen=iter_loss_window)
        self.total_training_time_s = 0.0
        self.timed_steps = 0
        self.train_batches_consumed = 0
        self._validation_batches: list[tuple[torch.Tensor, torch.Tensor]] = []
        self.tokens_per_iter = 0
        self.world_size = getattr(engine, "data_parallel_world_size", 1)
        self.global_tokens_per_iter = 0
        self.last_step_loss: float | None = None
        if fused_loss is None:
            fused_loss = bool(getattr(_unwrap(model), "supports_fused_loss", False))
        self.fused_loss = fused_loss
        if self.flops_per_token is None:
            self.flops_per_token = self._infer_flops_per_token()
        if self.peak_flops is None:
            self.peak_flops = self._infer_peak_flops()

    # -- helpers -------------------------------------------------------------------------------
    def _maybe_cudagraph_step_begin(self) -> None:
        if self.cudagraph_mark_step_begin and hasattr(torch.compiler, "cudagraph_mark_step_begin"):
            torch.compiler.cudagraph_mark_step_begin()

    @staticmethod
    def _is_distributed() -> bool:
        return dist.is_available() and dist.is_initialized()

    def _all_reduce_sum(self, tensor: torch.Tensor) -> torch.Tensor:
        if self._is_distributed():
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
        return tensor

    def _infer_flops_per_token(self) -> float | None:
        model = _unwrap(self.model)
        if hasattr(model, "estimate_flops"):
            try:
                return float(model.estimate_flops())
            except Exception:
                pass
        try:
            return float(6.0 * sum(p.numel() for p in model.parameters() if p.requires_grad))
        except Exception:
            return None

    def _infer_peak_flops(self) -> float | None:
        device = self.engine.device
        if device.type != "cuda" or not torch.cuda.is_available():
            return None
        index = device.index if device.index is not None else torch.cuda.current_device()
        name = torch.cuda.get_device_name(index).upper()
        if "B200" in name:
            measured = measured_peak_flops()
            if measured:
                return measured
        for key, value in PEAK_BF16_FLOPS.items():
            if key in name:
                return value
        return None

    def _compute_perf_metrics(self, idx: int, elapsed_time: float):
        tokens_per_sec = self.global_tokens_per_iter / max(elapsed_time, 1e-9)
        mfu = None
        if self.flops_per_token and self.peak_flops:
            denom = self.peak_flops * max(1, self.world_size)
            if denom > 0:
                mfu = 100.0 * self.flops_per_token * tokens_per_sec / denom
        if idx > self.timing_warmup_steps:
            self.total_training_time_s += elapsed_time
            self.timed_steps += 1
        eta_seconds = avg_step = None
        if self.timed_steps > 0:
            avg_step = self.total_training_time_s / self.timed_steps
            eta_seconds = max(self.max_iters - idx, 0) * avg_step
        return tokens_per_sec, mfu, eta_seconds, avg_step

    # -- evaluation ----------------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self, dataloader: DataLoader, num_batches: int) -> dict[str, float]:
        was_training = self.model.training
        self.model.eval()
        wanted = max(1, int(num_batches))
        is_validation = dataloader is self.val_dataloader
        iterator: Any
        if is_validation and len(self._validation_batches) >= wanted:
            iterator = iter(self._validation_batches[:wanted])
        else:
            # Never advance a persistent iterator: evaluate on a throw-away cycle of the source.
            source = dataloader.iterable if isinstance(dataloader, BetterCycle) else dataloader
            iterator = BetterCycle(source)
            if is_validation:
                self._validation_batches = [
                    self.engine.to_device(next(iterator)) for _ in range(wanted)
                ]
                iterator.close()
                gc.collect()
                iterator = iter(self._validation_batches)

        device = self.engine.device
        sums = {
            key: torch.zeros((), device=device, dtype=torch.float64)
            for key in ("loss", "tokens", "correct", "bpb_nats", "bytes")
        }
        for _ in range(wanted):
            data, target = self.engine.to_device(next(iterator))
            self._maybe_cudagraph_step_begin()
            with self.engine.autocast_context():
                logits: torch.Tensor = self.model(data)
            flat_logits = logits.float().reshape(-1, logits.size(-1))
            flat_target = target.reshape(-1)
            valid = flat_target != self.ignore_index
            valid_count = valid.sum()
            if valid_count.item() == 0:
                continue
            token_losses = F.cross_entropy(
                flat_logits, flat_target, ignore_index=self.ignore_index, reduction="none"
            )
            correct = (flat_logits.argmax(dim=-1).eq(flat_target) & valid).sum()
            if self.token_bytes is not None:
                if self.token_bytes.numel() < flat_logits.size(-1):
                    raise ValueError("token_bytes is smaller than the model vocabulary")
                safe_target = torch.where(valid, flat_target, torch.zeros_like(flat_target))
                byte_counts = self.token_bytes[safe_target]
                counted = valid & byte_counts.gt(0)
                sums["bpb_nats"] += token_losses[counted].sum()
                sums["bytes"] += byte_counts[counted].sum()
            sums["loss"] += token_losses.sum()
            sums["tokens"] += valid_count
            sums["correct"] += correct

        if isinstance(iterator, BetterCycle):
            iterator.close()
            gc.collect()
        for value in sums.values():
            self._all_reduce_sum(value)
        tokens = float(sums["tokens"].item())
        if was_training:
            self.model.train()
        if tokens <= 0:
            raise RuntimeError("evaluation produced no valid target tokens")
        mean_loss = float((sums["loss"] / tokens).item())
        metrics = {
            "loss": mean_loss,
            "ppl": float(math.exp(mean_loss)),
            "bits_per_token": float(mean_loss / math.log(2)),
            "accuracy": float((sums["correct"] / tokens).item()),
            "tokens": tokens,
        }
        if self.token_bytes is not None:
            total_bytes = float(sums["bytes"].item())
            metrics["bpb"] = (
                float(sums["bpb_nats"].item()) / (math.log(2) * total_bytes)
                if total_bytes > 0 else float("inf")
            )
            metrics["bytes"] = total_bytes
        return metrics

    @torch.no_grad()
    def calculate_loss(self, dataloader: DataLoader, num_batches: int) -> torch.Tensor:
        return torch.tensor(self.evaluate(dataloader, num_batches)["loss"], device=self.engine.device)

    def log_function(self, idx: int, lr: float, elapsed_time: float,
                     train_step_loss: float | None = None, tokens_per_sec: float | None = None,
                     mfu: float | None = None, eta_seconds: float | None = None) -> None:
        train_eval = (
            self.evaluate(self.train_dataloader, self.eval_train_batches)
            if self.eval_train_batches > 0 else None
        )
        val_eval = self.evaluate(self.val_dataloader, self.eval_val_batches)
        parts = [f"iter: {idx}"]
        if train_eval is not None:
            parts += [f"train_loss: {train_eval['loss']:.4f}", f"train_ppl: {train_eval['ppl']:.2f}"]
        parts += [f"val_loss: {val_eval['loss']:.4f}", f"val_ppl: {val_eval['ppl']:.2f}",
                  f"val_bits/token: {val_eval['bits_per_token']:.4f}"]
        if "bpb" in val_eval:
            parts.append(f"val_bpb: {val_eval['bpb']:.4f}")
        parts += [f"val_acc: {val_eval['accuracy']:.4f}", f"lr: {lr:e}", f"time: {elapsed_time:.4f}s"]
        if tokens_per_sec is not None:
            parts.append(f"tok/s: {tokens_per_sec:,.0f}")
        if mfu is not None:
            parts.append(f"mfu: {mfu:.2f}%")
        if eta_seconds is not None:
            parts.append(f"eta: {eta_seconds / 60.0:.1f}m")
        if self.engine.is_global_zero:
            print(" | ".join(parts))

        logs: dict[str, float] = {
            "validation_loss": val_eval["loss"],
            "validation_ppl": val_eval["ppl"],
            "validation_bits_per_token": val_eval["bits_per_token"],
            "validation_accuracy": val_eval["accuracy"],
            "iter": idx,
            "tokens": idx * self.global_tokens_per_iter,
            "lr": lr,
            "time": elapsed_time,
            "total_training_time_s": self.total_training_time_s,
        }
        if "bpb" in val_eval:
            logs["validation_bpb"] = val_eval["bpb"]
        if train_eval is not None:
            logs.update(
                training_eval_loss=train_eval["loss"], training_eval_ppl=train_eval["ppl"],
                training_eval_bits_per_token=train_eval["bits_per_token"],
                training_eval_accuracy=train_eval["accuracy"],
            )
        optional = {"training_step_loss": train_step_loss, "tokens_per_sec": tokens_per_sec,
                    "mfu": mfu, "eta_seconds": eta_seconds}
        logs.update({k: float(v) for k, v in optional.items() if v is not None})
        try:
            self.engine.log_dict(logs, step=idx)
        except Exception as error:
            print(f"Error logging: {error}")

    # -- one optimizer step --------------------------------------------------------------------
    def _apply_schedules(self, idx: int) -> float:
        lr = self.get_lr(idx)
        if not math.isfinite(lr) or lr < 0:
            raise RuntimeError(f"invalid learning rate at iter={idx}: {lr}")
        for group in self.optimizer.param_groups:
            group["lr"] = lr * float(group.get("lr_scale", 1.0))
        if self.get_optimizer_hparams is not None:
            hparams = self.get_optimizer_hparams(idx)
            unknown = set(hparams) - {"momentum", "weight_decay"}
            if unknown:
                raise ValueError(
                    "unknown scheduled optimizer hyperparameters: " + ", ".join(sorted(unknown))
                )
            for group in self.optimizer.param_groups:
                if group.get("kind") != "muon":
                    continue
                for key in ("momentum", "weight_decay"):
                    if key in hparams:
                        group[key] = float(hparams[key])
        return lr

    def _section(self, name: str):
        return self.timer.section(name) if self.timer is not None else nvtx_range(name)

    def section_times(self, reset: bool = True) -> dict[str, dict[str, float]]:
        """Milliseconds per phase (``forward_backward``, ``clip``, ``optimizer``) accumulated since
        the last reset, the maximum over ranks; empty unless ``profile_sections`` was set."""
        if self.timer is None:
            return {}
        summary = self.timer.summary()
        if reset:
            self.timer.reset()
        return summary

    def _micro_step_loss(self, data: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Σ cross-entropy over the supervised targets of one micro-batch (fp32 scalar)."""
        with self.engine.autocast_context():
            if self.fused_loss:
                return self.model(data, targets=target, ignore_index=self.ignore_index)
            logits: torch.Tensor = self.model(data)
            return F.cross_entropy(
                logits.float().reshape(-1, logits.size(-1)), target.reshape(-1),
                ignore_index=self.ignore_index, reduction="sum",
            )

    def train_step(self, idx: int) -> tuple[float, float]:
        """Run iteration ``idx`` (1-based). Returns ``(step_loss, lr)``."""
        lr = self._apply_schedules(idx)
        batches = [self.engine.to_device(next(self.train_dataloader)) for _ in range(self.micro_batch)]
        self.train_batches_consumed += self.micro_batch
        total_valid = sum((target != self.ignore_index).sum() for _, target in batches)
        inv_valid = 1.0 / total_valid.clamp_min(1).to(torch.float32)
        loss_sum_total = torch.zeros((), device=self.engine.device, dtype=torch.float32)
        for micro_step, (data, target) in enumerate(batches):
            if self.tokens_per_iter == 0:
                self.tokens_per_iter = int(data.numel() * self.micro_batch)
                self.global_tokens_per_iter = self.tokens_per_iter * self.world_size
            sync = (
                self.engine.no_backward_sync(self.model, enabled=micro_step < self.micro_batch - 1)
                if self.micro_batch > 1 else nullcontext()
            )
            with sync, self._section("train.forward_backward"):
                self._maybe_cudagraph_step_begin()
                loss_sum = self._micro_step_loss(data, target)
                loss_sum_total += loss_sum.detach().float()
                self.engine.backward(loss_sum * inv_valid)
        # One host read covers the three guards of the step: supervised tokens exist, every
        # micro-batch loss was finite (a non-finite term makes the sum non-finite).
        valid_host, loss_host = torch.stack([total_valid.float(), loss_sum_total]).tolist()
        if valid_host == 0:
            raise RuntimeError(f"training batch at iter={idx} has no valid target tokens")
        if not math.isfinite(loss_host):
            raise RuntimeError(f"Non-finite loss detected at iter={idx}: {loss_host}")
        if self.grad_clip_norm is not None and self.grad_clip_norm > 0:
            with self._section("train.clip"):
                grad_norm = self.engine.clip_gradients(self.model, self.optimizer,
                                                       max_norm=float(self.grad_clip_norm))
            if not torch.isfinite(grad_norm):
                raise RuntimeError(
                    f"Non-finite gradient norm detected at iter={idx}: {float(grad_norm)}"
                )
        with self._section("train.optimizer"):
            self.engine.optimizer_step(self.optimizer)
            self.optimizer.zero_grad(set_to_none=True)
            if self.apply_router_balancing is not None:
                self.apply_router_balancing(self.model)
        step_loss = loss_host / valid_host
        self.last_step_loss = step_loss
        return step_loss, lr

    # -- the loop ------------------------------------------------------------------------------
    def train(self, start_iter: int = 0):
        self.engine.launch()
        if not 0 <= start_iter <= self.max_iters:
            raise ValueError("start_iter must be between 0 and max_iters")
        self.model.train()
        self.optimizer.zero_grad(set_to_none=True)
        idx = start_iter
        while idx < self.max_iters:
            idx += 1
            self.engine.synchronize()
            check_peers = getattr(self.engine, "check_peers", None)
            if callable(check_peers):
                check_peers()  # raises before anything is launched that would wait on a lost rank
            guard = getattr(self.engine, "guard_step", None)
            started = time.perf_counter()
            with guard(idx) if callable(guard) else nullcontext():
                step_loss, lr = self.train_step(idx)
                self.engine.synchronize()
            elapsed = time.perf_counter() - started
            self._check_device_status()  # a kernel that abandoned a wait left stale data behind
            tokens_per_sec, mfu, eta_seconds, _ = self._compute_perf_metrics(idx, elapsed)
            if idx % self.print_every == 0 and self.engine.is_global_zero:
                line = (f"iter: {idx} | loss: {step_loss:.4f} | lr: {lr:e} | time: {elapsed:.4f}s "
                        f"| tok/s: {tokens_per_sec:,.2f}")
                if mfu is not None:
                    line += f" | mfu: {mfu:.2f}%"
                if eta_seconds is not None:
                    line += f" | eta: {eta_seconds / 60.0:.1f}m"
                print(line)
            if self.log_iter_loss:
                self.iter_loss_history.append(step_loss)
                try:
                    self.engine.log_dict(
                        {
                            "train_iter_loss": step_loss,
                            "train_iter_loss_100": sum(self.iter_loss_history) / len(self.iter_loss_history),
                            "iter": idx,
                            "tokens": idx * self.global_tokens_per_iter,
                            "lr": lr,
                            "time": elapsed,
                            "tokens_per_sec": tokens_per_sec,
                            "total_training_time_s": self.total_training_time_s,
                        },
                        step=idx,
                    )
                except Exception as error:
                    print(f"Error logging iter loss: {error}")
            last = idx == self.max_iters
            if self.eval_iters > 0 and (idx % self.eval_iters == 0 or last):
                self.model.eval()
                self.log_function(idx=idx, lr=lr, elapsed_time=elapsed, train_step_loss=step_loss,
                                  tokens_per_sec=tokens_per_sec, mfu=mfu, eta_seconds=eta_seconds)
                self.model.train()
            if self.save_ckpt_iters > 0 and (idx % self.save_ckpt_iters == 0 or last):
                self.save_checkpoint(idx, lr, step_loss)
        self.close()

    def checkpoint_state(self, idx: int, lr: float, step_loss: float) -> dict[str, Any]:
        full_state = getattr(self.engine, "full_state_dict", None)
        model_state = full_state(self.model) if callable(full_state) else self.model.state_dict()
        state = {
            "model": model_state,
            "optimizer": (self.engine.optimizer_state_dict(self.optimizer)
                          if callable(getattr(self.engine, "optimizer_state_dict", None))
                          else self.optimizer.state_dict()),
            "idx": idx,
            "lr": lr,
            "train_step_loss": step_loss,
            "gradient_accumulation_steps": self.micro_batch,
            "train_batches_consumed": self.train_batches_consumed,
            "torch_rng_state": torch.get_rng_state(),
        }
        if torch.cuda.is_available():
            state["cuda_rng_state_all"] = torch.cuda.get_rng_state_all()
        return state

    def _check_device_status(self) -> None:
        check = getattr(self.engine, "check_device_status", None)
        if callable(check):
            check()

    def save_checkpoint(self, idx: int, lr: float, step_loss: float) -> None:
        self.engine.synchronize()
        self._check_device_status()  # never persist weights that a timed-out collective left stale
        self.engine.save(self.checkpoint_path, self.checkpoint_state(idx, lr, step_loss))
        config = getattr(_unwrap(self.model), "config", None)
        if config is not None:
            config.ckpt_iter = idx
        if self.push_to_hub:
            self.model.push_to_hub(self.model_name, commit_message=f"checkpoint iter: {idx}")

    def close(self) -> None:
        """Release streaming iterators before interpreter shutdown."""
        self.train_dataloader.close()
        self.val_dataloader.close()
        gc.collect()
