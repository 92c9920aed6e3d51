"""Training throughput benchmarks: tokens/s of one optimizer step of the named configuration.

    python bench.py --gpus N --steps K --warmup W                    # depth-12 pretraining (default)
    python bench.py --config tp4_fsdp2_1p3b --gpus 8 ...             # another configuration
    python bench.py --impl reference --gpus N --steps K ...          # the reference arm

Configurations (``--config``; every one uses synthetic uniform-random tokens and random-init
weights, bf16 compute with fp32 master weights, and is weak-scaled: the work per data-parallel
replica is fixed, ``value`` is the whole-job tokens/s):

``d12`` (default)
    12 layers, d_model 768, 6 heads x 128, SwiGLU hidden 2048, vocab 50304, sequence 2048,
    32 sequences per GPU; Muon on the hidden matrices + AdamW on embeddings / head / norms;
    sharded optimizer with fused NVLink collectives over all N GPUs.
``tp4_fsdp2_1p3b``
    24 layers, d_model 2048, 16 query / 4 KV heads x 128, SwiGLU hidden 5632, vocab 50304,
    sequence 4096, 128 sequences per data-parallel replica and step (256 at 8 GPUs) in
    micro-batches of 16; AdamW; tensor parallel (sequence-parallel layout, collectives fused into
    the GEMMs) of degree min(4, N) x sharded optimizer over the rest.
``fsdp_1p3b`` / ``fsdp_1p3b_sharded_parameters``
    the same 1.3B model under plain data parallelism (4 sequences of 4096 x 4 micro-batches per
    GPU; AdamW): sharded optimizer with full parameters on every GPU, or the parameters themselves
    sharded per block and gathered just in time (``EngineConfig(shard_parameters=True)``); the
    JSON line of the second carries the parameter bytes a rank keeps and the most it gathered.
``cp8_32k``
    the same 1.3B model at sequence 32768, one sequence per context-parallel group and step;
    context parallel over all N GPUs (zig-zag shards, KV exchange under flash attention), sharded
    optimizer over the same ranks.
``moe_ep8`` / ``moe_ep8_skewed``
    16 layers, d_model 1024, 16 heads x 64, 64 routed SwiGLU experts (hidden 512) top-8 softmax
    router + a shared expert of hidden 1024 per layer, capacity factor 1.25, auxiliary
    load-balance loss 0.01, vocab 50304, sequence 2048, 16 sequences per GPU; AdamW; expert
    parallel over all N GPUs, sharded optimizer for the dense parameters. ``_skewed`` forces
    half of every token's picks onto four experts per layer (eight over the model, all on the
    first expert-parallel rank): 8 experts take 50 % of the picks.
``sft_d12``
    the depth-12 model on chat rows: synthetic conversations (2-6 alternating turns of 16-256
    tokens, wrapped in the chat special tokens) rendered with an assistant-only loss mask and
    best-fit packed into rows of 2048 by the package's own ``ConversationDataset``.

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``;
RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* come from the environment. Rank 0 prints one JSON line.

Two measurements per run, both through the public API (``Trainer.train_step``), both timed on the
device with CUDA events between barrier + synchronize, max over ranks:
  * ``value``: batches already resident on the device (no host->device traffic in the timed region);
  * ``e2e``  : every step copies its inputs from pinned host memory and reads the loss back.

``OHARA_BENCH_TP=k`` overrides the tensor-parallel degree of ``tp4_fsdp2_1p3b`` (to exercise tensor
parallel x sharded optimizer on fewer than eight GPUs). ``--tiny`` shrinks every configuration to a toy size (also runs on CPU / gloo): a functional check
of the plumbing, never a benchmark number; the JSON line then carries ``"tiny": true``.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import random
import shutil
import statistics
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent

LLAMA_1P3B = dict(num_layers=24, hidden_size=2048, num_heads=16, num_kv_heads=4,
                  intermediate_size=5632, vocab_size=50304)

CONFIGS: dict[str, dict] = {
    "d12": dict(
        name="llama-depth12 (12L d768 6hx128 ffn2048 V50304)",
        model=dict(num_layers=12, hidden_size=768, num_heads=6, num_kv_heads=0,
                   intermediate_size=2048, vocab_size=50304),
        seq_len=2048, rows=32, micro_steps=1, optimizer="muon_adamw", data="uniform",
    ),
    "tp4_fsdp2_1p3b": dict(
        name="llama-1.3B (24L d2048 16q/4kv x128 ffn5632 V50304)",
        model=LLAMA_1P3B, seq_len=4096, rows=16, micro_steps=8, optimizer="adamw", data="uniform",
        tp=4,
    ),
    "cp8_32k": dict(
        name="llama-1.3B (24L d2048 16q/4kv x128 ffn5632 V50304) @ 32k",
        model=LLAMA_1P3B, seq_len=32768, rows=1, micro_steps=1, optimizer="adamw", data="uniform",
        cp="all",
    ),
    "moe_ep8": dict(
        name="llama-moe (16L d1024 16hx64, 64 x h512 top-8 + shared h1024, V50304)",
        model=dict(num_layers=16, hidden_size=1024, num_heads=16, num_kv_heads=0,
                   intermediate_size=512, vocab_size=50304, moe_num_experts=64,
                   moe_experts_per_tok=8, moe_num_shared_experts=2, moe_gate_fn="softmax",
                   moe_aux_loss_coef=0.01, moe_capacity_factor=1.25),
        seq_len=2048, rows=16, micro_steps=1, optimizer="adamw", data="uniform", ep="all",
    ),
    "sft_d12": dict(
        name="llama-depth12 (12L d768 6hx128 ffn2048 V50304), chat SFT rows",
        model=dict(num_layers=12, hidden_size=768, num_heads=6, num_kv_heads=0,
                   intermediate_size=2048, vocab_size=50304),
        seq_len=2048, rows=32, micro_steps=1, optimizer="muon_adamw", data="chat",
    ),
}
CONFIGS["fsdp_1p3b"] = dict(
    name="llama-1.3B (24L d2048 16q/4kv x128 ffn5632 V50304), data parallel",
    model=LLAMA_1P3B, seq_len=4096, rows=4, micro_steps=4, optimizer="adamw", data="uniform",
)
CONFIGS["fsdp_1p3b_sharded_parameters"] = dict(CONFIGS["fsdp_1p3b"], shard_parameters=True,
                                               name=CONFIGS["fsdp_1p3b"]["name"]
                                               + ", parameters sharded per block")
CONFIGS["moe_ep8_skewed"] = dict(CONFIGS["moe_ep8"], skewed=True,
                                 name=CONFIGS["moe_ep8"]["name"] + ", skewed router (half of each token's picks forced onto experts of one rank)")

TINY_MODEL = dict(num_layers=2, hidden_size=64, num_heads=4, intermediate_size=64, vocab_size=512)

# kept for the reference arm of the default configuration
MODEL = dict(CONFIGS["d12"]["model"], name=CONFIGS["d12"]["name"], seq_len=2048, batch_per_gpu=32)

OPTIMIZER_LABELS = {
    "muon_adamw": "Muon (5 Newton-Schulz steps) on hidden matrices + AdamW on embeddings / head / norms",
    "adamw": "AdamW lr 3e-4 betas (0.9, 0.95) wd 0.1",
}
PRECISION_LABEL = "bf16 autocast, fp32 master weights"


def resolve(name: str, world: int, tiny: bool) -> dict:
    """Concrete workload of configuration ``name`` on ``world`` GPUs: model settings, parallel
    degrees (``tp``, ``cp``, ``ep``; the remaining factor is data parallel), rows per micro-batch
    of one data-parallel replica, micro-batches per step."""
    spec = dict(CONFIGS[name])
    spec["key"] = name
    model = dict(spec["model"])
    if tiny:
        keep = {k: v for k, v in model.items() if k.startswith("moe_")}
        model = dict(TINY_MODEL, num_kv_heads=2 if model.get("num_kv_heads") else 0, **keep)
        if keep:
            model.update(moe_num_experts=8, moe_experts_per_tok=2, intermediate_size=32)
        spec["seq_len"] = 256 if spec["seq_len"] > 4096 else 128
        spec["rows"] = min(spec["rows"], 4)
        spec["micro_steps"] = min(spec["micro_steps"], 2)
    spec["model"] = model
    tp = math.gcd(int(os.environ.get("OHARA_BENCH_TP", spec.get("tp", 1))), world)
    cp = world // tp if spec.get("cp") == "all" else 1
    ep = world // (tp * cp) if spec.get("ep") == "all" else 1
    spec.update(tp=tp, cp=cp, ep=ep, dp=world // (tp * cp * ep))
    parts = [f"{k}{spec[k]}" for k in ("tp", "cp", "ep") if spec[k] > 1]
    if spec["dp"] > 1 or not parts:
        parts.append(f"fsdp{spec['dp']}" if world > 1 else "single")
    spec["parallelism"] = " x ".join(parts)
    return spec


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


# --------------------------------------------------------------------------------------------------
# Synthetic chat data (both arms build their own ConversationDataset from these)
# --------------------------------------------------------------------------------------------------
class IdTokenizer:
    """Tokenizer whose "text" is a space-separated list of token ids, so that synthetic
    conversations of exact token lengths can go through the real rendering and packing code. The
    chat special tokens take the highest ids of the vocabulary."""

    SPECIALS = ("<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>",
                "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>")

    def __init__(self, vocab_size: int) -> None:
        self.vocab_size = vocab_size
        self.name_or_path = "synthetic-ids"
        self._special = {token: vocab_size - 1 - i for i, token in enumerate(self.SPECIALS)}
        self.bos_token_id = vocab_size - 1 - len(self.SPECIALS)
        self.eos_token_id = self.pad_token_id = self.bos_token_id
        self.first_special = self.bos_token_id
        self.padding_side = "right"

    def __len__(self) -> int:
        return self.vocab_size

    def get_vocab(self) -> dict[str, int]:
        return dict(self._special)

    def convert_tokens_to_ids(self, token: str):
        return self._special.get(token)

    def add_special_tokens(self, mapping) -> int:
        return 0

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return [int(piece) for piece in text.split()]

    def __call__(self, texts, add_special_tokens: bool = False, **_):
        if isinstance(texts, str):
            return {"input_ids": self.encode(texts)}
        return {"input_ids": [self.encode(t) for t in texts]}


def synthetic_conversations(count: int, vocab_size: int, seed: int) -> list[dict]:
    """``count`` conversations of 2-6 alternating user / assistant turns, each turn 16-256
    uniform-random ordinary tokens."""
    rng = random.Random(seed)
    limit = IdTokenizer(vocab_size).first_special
    conversations = []
    for _ in range(count):
        turns = rng.randint(2, 6)
        messages = []
        for turn in range(turns):
            length = rng.randint(16, 256)
            text = " ".join(str(rng.randrange(limit)) for _ in range(length))
            messages.append({"role": "user" if turn % 2 == 0 else "assistant", "content": text})
        conversations.append({"messages": messages})
    return conversations


def force_router_skew(model, moe_class, top_k: int) -> dict:
    """Force half of every token's top-k picks onto a few experts: in every mixture-of-experts
    layer of ``model`` the selection bias of ``top_k // 2`` experts is raised far above any logit
    (experts ``0 .. k/2-1`` in even layers, ``k/2 .. k-1`` in odd ones), so each token picks those
    and fills its other slots by the learned router. Over the model the first ``top_k`` experts
    take half of all picks, each favoured expert ``experts / 2k`` times the mean load of its
    layer, and under expert parallelism they all live on the first rank.

    The construction does not depend on the logits. A moderate bias calibrated on the logits of a
    probe batch does not hold: with a learning rate of 3e-4 from step one the residual stream of a
    freshly initialised model changes direction within a few steps, the per-token spread of the
    router logits shrinks, and a share calibrated to 50 % was measured at 27 to 32 % over the
    following steps. Gate weights still come from the unbiased logits. Used by both arms;
    ``moe_class`` is the arm's own grouped mixture-of-experts module."""
    import torch

    half = max(top_k // 2, 1)
    layers = [m for m in model.modules() if isinstance(m, moe_class)]
    with torch.no_grad():
        for i, layer in enumerate(layers):
            first = half * (i % 2)
            layer.router_bias.zero_()
            layer.router_bias[first:first + half] = 1.0e3
    return {"favoured_experts_per_layer": half, "favoured_experts": 2 * half,
            "target_share": half / top_k, "bias": 1.0e3}


# --------------------------------------------------------------------------------------------------
# This framework
# --------------------------------------------------------------------------------------------------
def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist
    from torch.utils.data import DataLoader, IterableDataset

    import ohara_b200
    from ohara_b200 import Config, Llama, OharaEngine, Trainer
    from ohara_b200.lr_scheduler import Scheduler
    from ohara_b200.optimizer import build_adamw, build_muon_adamw
    from ohara_b200.runtime import EngineConfig, ParallelConfig, StrategyType, TensorParallelPlan

    rank = int(os.environ.get("RANK", "0"))
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    spec = resolve(args.config, world_env, args.tiny)
    torch.manual_seed(1234 + rank)
    strategy = StrategyType.FSDP if world_env > 1 else StrategyType.SINGLE
    engine = OharaEngine(EngineConfig(
        strategy=strategy,
        parallel=ParallelConfig(tp=spec["tp"], cp=spec["cp"], ep=spec["ep"]),
        # sequence-parallel layout with the collectives inside the GEMMs (needs the GPUs)
        tensor_parallel=TensorParallelPlan.llama_default(
            spec["tp"], sequence_parallel=torch.cuda.is_available())
        if spec["tp"] > 1 else TensorParallelPlan(),
        expert_capacity_factor=1.25 if spec["ep"] > 1 else 2.0,
        shard_parameters=bool(spec.get("shard_parameters")) and world_env > 1,
        # the key/value exchange under the flash kernels needs peer memory; CPU ranks (functional
        # checks at toy size) cut the sequence the same way and exchange with all-to-alls
        context_parallel_mode="ring" if torch.cuda.is_available() else "ulysses",
    ))
    engine.launch()
    device = engine.device
    on_gpu = device.type == "cuda"
    if not on_gpu and not args.tiny:
        raise SystemExit("bench.py needs a CUDA device")

    m = spec["model"]
    seq, rows, micro_steps, vocab = spec["seq_len"], spec["rows"], spec["micro_steps"], m["vocab_size"]
    moe = {k: v for k, v in m.items() if k.startswith("moe_")}
    if moe:
        moe["moe_grouped"] = True
    cfg = Config(
        vocab_size=vocab, max_sequence_length=seq, hidden_size=m["hidden_size"],
        intermediate_size=m["intermediate_size"], num_attention_heads=m["num_heads"],
        num_key_value_heads=m.get("num_kv_heads", 0), num_hidden_layers=m["num_layers"],
        dropout=0.0, weight_tying=False, rope_theta=10000.0, **moe,
    )
    model = engine.prepare(Llama(cfg))
    if spec["optimizer"] == "muon_adamw":
        base = build_muon_adamw(model)
        learning_rate = 0.02
    else:
        learning_rate = 3e-4
        base = build_adamw(model, learning_rate=learning_rate, weight_decay=0.1, betas=(0.9, 0.95))
    (optimizer,) = engine.prepare_optimizers(base)

    skew = None
    if spec.get("skewed"):
        # Half of every token's picks forced onto a few experts of the first rank; the
        # balancing update stays off so that the skew persists.
        from ohara_b200.modules.moe_grouped import GroupedMoE

        skew = force_router_skew(model, GroupedMoE, m["moe_experts_per_tok"])

    dp_rank, dp_world = engine.data_parallel_rank, engine.data_parallel_world_size

    def uniform_rows(gen):
        block = torch.randint(0, vocab, (rows, seq + 1), generator=gen)
        return block[:, :-1].contiguous(), block[:, 1:].contiguous()

    if spec["data"] == "chat":
        from ohara_b200.sft import ConversationDataset

        tokenizer = IdTokenizer(vocab)
        conversations = synthetic_conversations(4096 if not args.tiny else 64, vocab, seed=17)
        source = iter(ConversationDataset(conversations, tokenizer, max_length=seq, seed=5,
                                          data_rank=dp_rank, data_world_size=dp_world))

        def chat_rows(gen):
            pairs = [next(source) for _ in range(rows)]
            return (torch.stack([p[0] for p in pairs]).contiguous(),
                    torch.stack([p[1] for p in pairs]).contiguous())

        make_rows = chat_rows
    else:
        make_rows = uniform_rows

    pool_size = 4
    host_pool, device_pool = [], []
    gen = torch.Generator().manual_seed(99 + dp_rank)
    for _ in range(pool_size * micro_steps):
        x, y = make_rows(gen)
        host_pool.append((x.pin_memory(), y.pin_memory()) if on_gpu else (x, y))
    gen = torch.Generator().manual_seed(7 + dp_rank)
    for _ in range(pool_size * micro_steps):
        x, y = make_rows(gen)
        device_pool.append((x.to(device), y.to(device)))
    supervised = sum(int((y != -1).sum()) for _, y in host_pool) / max(1, len(host_pool))

    class Ring(IterableDataset):
        """Cycles over a pool of batches (device-resident, or pinned host memory)."""

        def __init__(self, pool):
            self.pool = pool

        def __iter__(self):
            i = 0
            while True:
                yield self.pool[i % len(self.pool)]
                i += 1

    balancing = None
    if moe and not spec.get("skewed"):
        from ohara_b200.modules.routing import apply_qb_update

        balancing = apply_qb_update

    def make_trainer(pool):
        loader = DataLoader(Ring(pool), batch_size=None)
        dl = engine.prepare_dataloaders(loader)
        return Trainer(engine, model, optimizer, dl, dl, Scheduler(learning_rate),
                       micro_batch=micro_steps, max_iters=10**9, eval_iters=0, save_ckpt_iters=0,
                       print_every=10**9, apply_router_balancing=balancing)

    def sync():
        if dist.is_initialized():
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    def launch_count() -> int:
        if not on_gpu:
            return 0
        from ohara_b200.ops._ext import ext

        return int(ext().launch_count())

    def timed(trainer, steps, first_idx, sampler=None):
        sync()
        launches0 = launch_count()
        if sampler:
            sampler.start()
        if on_gpu:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        else:
            import time

            began = time.perf_counter()
        for i in range(steps):
            trainer.train_step(first_idx + i)
        if on_gpu:
            stop.record()
        sync()
        clocks = sampler.stop() if sampler else None
        launches = launch_count() - launches0
        elapsed = start.elapsed_time(stop) if on_gpu else (time.perf_counter() - began) * 1e3
        ms = torch.tensor([elapsed], device=device, dtype=torch.float64)
        if dist.is_initialized():
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, launches, clocks

    model.train()
    optimizer.zero_grad(set_to_none=True)
    device_trainer = make_trainer(device_pool)
    host_trainer = make_trainer(host_pool)
    idx = 1
    for _ in range(args.warmup):
        device_trainer.train_step(idx)
        idx += 1
    host_trainer.train_step(idx)  # touch the host path once before timing it
    idx += 1
    if moe:
        from ohara_b200.modules.routing import expert_load

        expert_load(model)  # reset the counters: the reported load covers the timed steps only
    sampler = ClockSampler(device.index or 0) if on_gpu else None
    ms_device, launches, clocks = timed(device_trainer, args.steps, idx, sampler)
    idx += args.steps
    ms_e2e, _, _ = timed(host_trainer, args.steps, idx)
    engine.synchronize()
    engine.check_device_status()

    load = None
    if moe:
        from ohara_b200.modules.routing import expert_load

        counts = expert_load(model)
        if counts is not None:
            total = counts.float().sum(0)
            if dist.is_initialized():
                dist.all_reduce(total)
            top = total.topk(min(8, total.numel())).values.sum() / total.sum().clamp_min(1)
            load = {"share_of_top8_experts": float(top),
                    "max_over_mean": float(total.max() / total.mean().clamp_min(1e-9))}
            dropped = [mod.dropped_pairs for mod in model.modules()
                       if getattr(mod, "dropped_pairs", None) is not None]
            if dropped:
                lost = torch.stack([d.float() for d in dropped]).sum()
                if dist.is_initialized():
                    dist.all_reduce(lost)
                pairs = rows * seq * m["moe_experts_per_tok"] * dp_world * len(dropped)
                load["dropped_pair_fraction_last_step"] = float(lost) / pairs
    world = dist.get_world_size() if dist.is_initialized() else 1
    tokens_per_step = rows * seq * micro_steps * dp_world
    memory = torch.cuda.max_memory_allocated(device) / 2**30 if on_gpu else None
    result = {
        "impl": "ohara_b200",
        "spec": spec,
        "value": tokens_per_step / (ms_device / 1e3),
        "ms_per_step": ms_device,
        "e2e_value": tokens_per_step / (ms_e2e / 1e3),
        "e2e_ms_per_step": ms_e2e,
        "tokens_per_step": tokens_per_step,
        # what one rank copies: its tensor-parallel slice of the rows, its context-parallel shard
        "h2d_bytes_per_step": 2 * (rows // spec["tp"] if spec["tp"] > 1 else rows)
        * (seq // spec["cp"]) * 8 * micro_steps,
        "d2h_bytes_per_step": 8,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "loss": host_trainer.last_step_loss,
        "flops_per_token": float(model.estimate_flops(min(seq, cfg.max_sequence_length))),
        "supervised_tokens_per_batch": supervised,
        "skew": skew,
        "expert_load": load,
        "peak_memory_gib": memory,
        "parameter_memory": (model._param_sharding.memory_report()
                             if getattr(model, "_param_sharding", None) is not None else None),
        "world": world,
        "is_rank0": engine.is_global_zero,
        "version": getattr(ohara_b200, "__version__", "0"),
    }
    engine.close()
    return result


def config_block(spec: dict, world: int, optimizer_label: str) -> dict:
    return {
        "name": spec["key"], "model": spec["name"],
        "global_batch": spec["rows"] * spec["micro_steps"] * spec["dp"] * spec["ep"],
        "seq_len": spec["seq_len"], "parallelism": spec["parallelism"],
        "optimizer": optimizer_label, "precision": PRECISION_LABEL,
        "l2": "working set per step >> 126 MB L2, no flush needed",
    }


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--config", choices=sorted(CONFIGS), default="d12")
    parser.add_argument("--tiny", action="store_true", help="toy sizes, functional check only")
    args = parser.parse_args()
    if args.warmup < 3 and not args.tiny:
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
    if args.tiny:
        common["tiny"] = True
    spec = resolve(args.config, max(world, 1), args.tiny)
    if spec["data"] == "chat":
        common["data"] = ("synthetic conversations (uniform-random tokens, 2-6 turns of 16-256), "
                          "assistant-only loss mask, best-fit packed; random-init weights")
    optimizer_label = OPTIMIZER_LABELS[spec["optimizer"]]

    if args.impl == "reference":
        sys.path.insert(0, str(ROOT))
        from baseline.reference_bench import reference_available, run

        ok, why = reference_available(args.config)
        if not ok:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "config": {"name": args.config},
                                  "unavailable": why}))
            return
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        res = run(args, spec, ClockSampler(local_rank))
        if res["is_rank0"]:
            base = baseline_number()
            block = config_block(spec, world, optimizer_label)
            block["parallelism"] = res["parallelism"]
            block["composition"] = res.get("composition", "reference as shipped")
            line = {
                **common,
                "impl": "reference",
                "value": res["value"],
                "ms_per_step": res["ms_per_step"],
                "vs_baseline": (res["value"] / base) if base else None,
                "config": block,
                "e2e": {"value": res["e2e_value"], "unit": "tokens/s",
                        "ms_per_step": res["e2e_ms_per_step"],
                        "h2d_bytes_per_step": res["h2d_bytes_per_step"],
                        "d2h_bytes_per_step": res["d2h_bytes_per_step"]},
                "clocks": res["clocks"],
                "final_loss": res.get("loss"),
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
            "config": config_block(res["spec"], world, optimizer_label),
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
            "peak_memory_gib": res["peak_memory_gib"],
        }
        for key in ("skew", "expert_load", "parameter_memory"):
            if res.get(key):
                line[key] = res[key]
        if res["spec"]["data"] == "chat":
            line["supervised_tokens_per_batch"] = res["supervised_tokens_per_batch"]
        print(json.dumps(line))


if __name__ == "__main__":
    main()
