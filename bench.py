"""Headline benchmark: training tokens/s of the depth-12 Llama pretraining step.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N --steps K ...  # unmodified reference (baseline/_ref)

Model / config (both arms): 12 layers, d_model 768, 6 heads x 128, SwiGLU hidden 2048, vocab 50304,
sequence 2048, 32 sequences per GPU, bf16 compute with fp32 master weights, Muon on the hidden
matrices + AdamW on embeddings / head / norms, random init, synthetic uniform-random tokens. Weak
scaling: per-GPU work is fixed, ``value`` is the whole-job tokens/s.

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``;
RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* come from the environment. Rank 0 prints one JSON line.

Two measurements per run, both through the public API (``Trainer.train_step``), both timed on the
device with CUDA events between barrier + synchronize, max over ranks:
  * ``value``: batches already resident on the device (no host->device traffic in the timed region);
  * ``e2e``  : every step copies its inputs from pinned host memory and reads the loss back.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent

MODEL = {
    "name": "llama-depth12 (12L d768 6hx128 ffn2048 V50304)",
    "num_layers": 12,
    "hidden_size": 768,
    "num_heads": 6,
    "intermediate_size": 2048,
    "vocab_size": 50304,
    "seq_len": 2048,
    "batch_per_gpu": 32,
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = (
        "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
        "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc: subprocess.Popen | None = None
        self.path: str | None = None

    def start(self) -> None:
        if shutil.which("nvidia-smi") is None:
            return
        handle, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(handle)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return summary
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, max_clock = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in Path(self.path).read_text().splitlines():
                cells = [c.strip() for c in line.split(",")]
                if len(cells) < 9:
                    continue
                try:
                    clocks.append(float(cells[1]))
                    max_clock = float(cells[2])
                except ValueError:
                    continue
                for name, cell in zip(names, cells[5:9]):
                    if cell.lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.unlink(self.path)
            except OSError:
                pass
        if clocks:
            summary.update(sm_mhz=statistics.median(clocks), sm_max_mhz=max_clock,
                           reasons=sorted(reasons), samples=len(clocks))
        return summary


def baseline_number() -> float | None:
    """The reference publishes no throughput figure for this benchmark (BASELINE.json has an empty
    ``published`` table), so there is nothing to divide by."""
    try:
        published = json.loads((ROOT / "BASELINE.json").read_text()).get("published", {})
    except (OSError, ValueError):
        return None
    value = published.get("train_tokens_per_sec") if isinstance(published, dict) else None
    return float(value) if value else None


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from torch.utils.data import DataLoader, IterableDataset

    import ohara_b200
    from ohara_b200 import Config, Llama, OharaEngine, Trainer
    from ohara_b200.lr_scheduler import Scheduler
    from ohara_b200.ops._ext import ext
    from ohara_b200.optimizer import build_muon_adamw
    from ohara_b200.runtime import EngineConfig, StrategyType

    rank = int(os.environ.get("RANK", "0"))
    torch.manual_seed(1234 + rank)
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    strategy = StrategyType.FSDP if world_env > 1 else StrategyType.SINGLE
    engine = OharaEngine(EngineConfig(strategy=strategy))
    engine.launch()
    device = engine.device
    if device.type != "cuda":
        raise SystemExit("bench.py needs a CUDA device")

    cfg = Config(
        vocab_size=MODEL["vocab_size"], max_sequence_length=MODEL["seq_len"],
        hidden_size=MODEL["hidden_size"], intermediate_size=MODEL["intermediate_size"],
        num_attention_heads=MODEL["num_heads"], num_key_value_heads=0,
        num_hidden_layers=MODEL["num_layers"], dropout=0.0, weight_tying=False, rope_theta=10000.0,
    )
    model = engine.prepare(Llama(cfg))
    (optimizer,) = engine.prepare_optimizers(build_muon_adamw(model))
    batch, seq, vocab = MODEL["batch_per_gpu"], MODEL["seq_len"], MODEL["vocab_size"]

    class HostBatches(IterableDataset):
        """Uniform random token rows generated on the host, one pinned batch per step."""

        def __iter__(self):
            gen = torch.Generator().manual_seed(99 + rank)
            while True:
                rows = torch.randint(0, vocab, (batch, seq + 1), generator=gen)
                yield rows[:, :-1].contiguous().pin_memory(), rows[:, 1:].contiguous().pin_memory()

    class DeviceBatches(IterableDataset):
        """A small ring of batches already on the device."""

        def __init__(self):
            gen = torch.Generator().manual_seed(7 + rank)
            self.ring = []
            for _ in range(4):
                rows = torch.randint(0, vocab, (batch, seq + 1), generator=gen).to(device)
                self.ring.append((rows[:, :-1].contiguous(), rows[:, 1:].contiguous()))

        def __iter__(self):
            i = 0
            while True:
                yield self.ring[i % len(self.ring)]
                i += 1

    def make_trainer(dataset):
        loader = DataLoader(dataset, batch_size=None)
        dl = engine.prepare_dataloaders(loader)
        return Trainer(engine, model, optimizer, dl, dl, Scheduler(0.02), micro_batch=1,
                       max_iters=10**9, eval_iters=0, save_ckpt_iters=0, print_every=10**9)

    def sync():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def timed(trainer, steps, first_idx, sampler=None):
        sync()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ext().launch_count()
        if sampler:
            sampler.start()
        start.record()
        for i in range(steps):
            trainer.train_step(first_idx + i)
        stop.record()
        sync()
        clocks = sampler.stop() if sampler else None
        launches = ext().launch_count() - launches0
        ms = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
        if dist.is_initialized():
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, launches, clocks

    model.train()
    optimizer.zero_grad(set_to_none=True)
    device_trainer = make_trainer(DeviceBatches())
    host_trainer = make_trainer(HostBatches())
    idx = 1
    for _ in range(args.warmup):
        device_trainer.train_step(idx)
        idx += 1
    host_trainer.train_step(idx)  # touch the host path once before timing it
    idx += 1
    sampler = ClockSampler(device.index or 0)
    ms_device, launches, clocks = timed(device_trainer, args.steps, idx, sampler)
    idx += args.steps
    ms_e2e, _, _ = timed(host_trainer, args.steps, idx)
    from ohara_b200 import ops

    ops.check_status()
    world = dist.get_world_size() if dist.is_initialized() else 1
    tokens_per_step = batch * seq * world
    result = {
        "impl": "ohara_b200",
        "value": tokens_per_step / (ms_device / 1e3),
        "ms_per_step": ms_device,
        "e2e_value": tokens_per_step / (ms_e2e / 1e3),
        "e2e_ms_per_step": ms_e2e,
        "tokens_per_step": tokens_per_step,
        "h2d_bytes_per_step": 2 * batch * seq * 8,
        "d2h_bytes_per_step": 8,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "loss": host_trainer.last_step_loss,
        "flops_per_token": float(model.estimate_flops()),
        "parallelism": "single" if world == 1 else f"fsdp{world}",
        "is_rank0": engine.is_global_zero,
        "version": getattr(ohara_b200, "__version__", "0"),
    }
    engine.close()
    return result


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.steps < 1:
        parser.error("--steps must be at least 1")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        parser.error(f"--gpus {args.gpus} does not match WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        parser.error("for --gpus > 1 launch with `python -m torch.distributed.run --nproc-per-node N`")

    common = {
        "metric": "train tokens/sec",
        "unit": "tokens/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "higher_is_better": True,
        "scaling": "weak",
        "dtype": "bf16",
        "data": "synthetic uniform-random tokens, random-init weights",
    }

    if args.impl == "reference":
        sys.path.insert(0, str(ROOT))
        from baseline.reference_bench import reference_available, run

        ok, why = reference_available()
        if not ok:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        res = run(args, MODEL, ClockSampler(local_rank))
        if res["is_rank0"]:
            base = baseline_number()
            line = {
                **common,
                "impl": "reference",
                "value": res["value"],
                "ms_per_step": res["ms_per_step"],
                "vs_baseline": (res["value"] / base) if base else None,
                "config": {
                    "model": MODEL["name"], "global_batch": MODEL["batch_per_gpu"] * args.gpus,
                    "seq_len": MODEL["seq_len"], "parallelism": res["parallelism"],
                    "optimizer": "reference build_muon_adamw", "precision": "bf16 autocast, fp32 master",
                    "l2": "working set per step >> 126 MB L2, no flush needed",
                },
                "e2e": {"value": res["value"], "unit": "tokens/s",
                        "h2d_bytes_per_step": res["h2d_bytes_per_step"],
                        "d2h_bytes_per_step": res["d2h_bytes_per_step"]},
                "clocks": res["clocks"],
            }
            print(json.dumps(line))
        return

    res = run_ours(args)
    if res["is_rank0"]:
        base = baseline_number()
        peak = None
        try:
            peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
            peak = float(peaks["bf16_tflops_sustained"]) * 1e12
        except (OSError, ValueError, KeyError):
            pass
        per_gpu_tok_s = res["value"] / args.gpus
        line = {
            **common,
            "impl": "ohara_b200",
            "value": res["value"],
            "ms_per_step": res["ms_per_step"],
            "vs_baseline": (res["value"] / base) if base else None,
            "config": {
                "model": MODEL["name"], "global_batch": MODEL["batch_per_gpu"] * args.gpus,
                "seq_len": MODEL["seq_len"], "parallelism": res["parallelism"],
                "optimizer": "Muon (5 NS steps) + AdamW", "precision": "bf16 compute, fp32 master",
                "l2": "working set per step >> 126 MB L2, no flush needed",
            },
            "e2e": {"value": res["e2e_value"], "unit": "tokens/s",
                    "ms_per_step": res["e2e_ms_per_step"],
                    "h2d_bytes_per_step": res["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": res["d2h_bytes_per_step"]},
            "gpu_launches": res["gpu_launches"],
            "clocks": res["clocks"],
            "mfu_of_measured_sustained": (
                res["flops_per_token"] * per_gpu_tok_s / peak if peak else None
            ),
            "final_loss": res["loss"],
        }
        print(json.dumps(line))


if __name__ == "__main__":
    main()
