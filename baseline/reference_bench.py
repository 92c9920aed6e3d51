"""Reference arm of the training benchmarks.

Runs the *unmodified* reference package (``ohara``, installed from the read-only source tree into
``baseline/_ref`` with ``pip install --no-index --no-deps --target``) through its own public API:
``ohara.Llama`` / ``Config``, ``OharaEngine``, ``ohara.optimizer.build_muon_adamw`` / ``build_adamw``
and ``ohara.Trainer.train``. None of this package's models, kernels or engine is imported here. The
only additions are a stub ``lightning`` module that the reference imports for a parameter summary
and that is not installed on this image, and — for the configurations that the reference cannot
run by itself — the stock PyTorch compositions of ``baseline/compositions.py`` around its modules:

* ``d12`` / ``sft_d12``: the reference as shipped (single device, or its DDP strategy);
* ``tp4_fsdp2_1p3b``: the reference engine's own tensor-parallel plan (DTensor
  ``parallelize_module``) with the local head counts corrected, ``fully_shard`` over the
  data-parallel mesh instead of DDP;
* ``cp8_32k``: ``torch.distributed.tensor.experimental.context_parallel`` (ring SDPA) around the
  reference model, ``fully_shard`` over the same ranks;
* ``moe_ep8``: the reference ``GroupedMoE`` with its experts sharded over the ranks and
  ``all_to_all_single`` dispatch / combine around its ``torch._grouped_mm`` calls, DDP for the
  dense parameters.

Timing: ``Trainer.train`` is called for the warm-up iterations and once more (``start_iter`` =
warm-up) for the timed iterations, bracketed by a barrier + ``torch.cuda.synchronize()`` and CUDA
events; the maximum over ranks is reported. As in the other arm there are two measurements:
batches resident on the device (``value``) and batches copied from pinned host memory every step
(``e2e``).
"""

from __future__ import annotations

import contextlib
import io
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def reference_available(config: str = "d12") -> tuple[bool, str]:
    root = HERE / "_ref" / "ohara"
    if not root.is_dir():
        return False, "baseline/_ref/ohara is missing (reference not installed)"
    return True, ""


def _import_reference():
    for extra in (HERE / "stubs", HERE / "_ref"):
        if str(extra) not in sys.path:
            sys.path.insert(0, str(extra))


def run(args, spec: dict, clock_sampler) -> dict:
    _import_reference()
    import torch
    import torch.distributed as dist
    from torch.utils.data import DataLoader, IterableDataset

    from ohara import Config, Llama, Trainer  # the reference package
    from ohara.lr_scheduler import Scheduler
    from ohara.optimizer import build_adamw, build_muon_adamw

    sys.path.insert(0, str(HERE.parent))
    from baseline import compositions

    rank = int(os.environ.get("RANK", "0"))
    torch.manual_seed(1234 + rank)
    torch.set_float32_matmul_precision("high")  # as examples/train_llama_engine.py:226 does
    engine, composition = compositions.build_engine(spec)
    engine.launch()
    device = engine.device
    on_gpu = device.type == "cuda"

    m = spec["model"]
    seq, rows, micro_steps, vocab = spec["seq_len"], spec["rows"], spec["micro_steps"], m["vocab_size"]
    # only the mixture-of-experts settings the reference Config knows (it has neither a capacity
    # factor nor an auxiliary loss: its experts are dropless and balanced by the router bias)
    moe = {k: v for k, v in m.items()
           if k in ("moe_num_experts", "moe_experts_per_tok", "moe_num_shared_experts", "moe_gate_fn")}
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
        optimizer = build_muon_adamw(model)
        learning_rate = 0.02
    else:
        learning_rate = 3e-4
        optimizer = build_adamw(model, learning_rate=learning_rate, weight_decay=0.1,
                                betas=(0.9, 0.95))

    if any(type(p).__name__ == "DTensor" for p in model.parameters()) and not all(
            type(p).__name__ == "DTensor" for p in model.parameters()):
        # tensor parallel without a sharded data-parallel dimension leaves plain tensors next to
        # DTensors, which the multi-tensor optimizer path cannot mix
        for group in optimizer.param_groups:
            group["foreach"] = False
    dp_rank, dp_world = compositions.data_rank(engine)

    def uniform_rows(gen):
        block = torch.randint(0, vocab, (rows, seq + 1), generator=gen)
        return block[:, :-1].contiguous(), block[:, 1:].contiguous()

    if spec["data"] == "chat":
        from ohara.sft import ConversationDataset  # the reference's renderer and packer

        from bench import IdTokenizer, synthetic_conversations

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

    class Ring(IterableDataset):
        def __init__(self, pool):
            self.pool = pool

        def __iter__(self):
            i = 0
            while True:
                yield self.pool[i % len(self.pool)]
                i += 1

    balancing = None
    if moe and not spec.get("skewed"):
        from ohara.modules.moe import apply_qb_update  # reference: once per optimizer step

        balancing = apply_qb_update
    if spec.get("skewed"):
        compositions.apply_router_skew(model, spec, cfg, device)

    def make_trainer(pool):
        loader = DataLoader(Ring(pool), batch_size=None)
        train_dl, val_dl = engine.prepare_dataloaders(loader, loader)
        return Trainer(
            engine, model, optimizer, train_dl, val_dl, Scheduler(learning_rate),
            micro_batch=micro_steps, max_iters=1, eval_iters=0, save_ckpt_iters=0,
            print_every=1, flops_per_token=1.0, peak_flops=1.0,
            apply_router_balancing=balancing,
        )

    def sync():
        if dist.is_initialized():
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize()

    def timed(trainer, first, steps, sampler=None):
        trainer.max_iters = first + steps
        sync()
        if sampler is not None:
            sampler.start()
        if on_gpu:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        else:
            import time

            began = time.perf_counter()
        trainer.train(start_iter=first)
        if on_gpu:
            stop.record()
        sync()
        clocks = sampler.stop() if sampler is not None else None
        elapsed = start.elapsed_time(stop) if on_gpu else (time.perf_counter() - began) * 1e3
        ms = torch.tensor([elapsed], device=device, dtype=torch.float64)
        if dist.is_initialized():
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, clocks

    quiet = io.StringIO()
    device_trainer, host_trainer = make_trainer(device_pool), make_trainer(host_pool)
    final_loss = None
    with contextlib.redirect_stdout(quiet):
        device_trainer.max_iters = max(args.warmup, 1)
        device_trainer.train(start_iter=0)
        host_trainer.max_iters = args.warmup + 1
        host_trainer.train(start_iter=args.warmup)  # touch the host path once before timing it
        ms_device, clocks = timed(device_trainer, args.warmup + 1, args.steps, clock_sampler)
        ms_e2e, _ = timed(host_trainer, args.warmup + 1 + args.steps, args.steps)
    for line in reversed(quiet.getvalue().splitlines()):
        if "loss:" in line:  # "iter: N | loss: X | ..."
            try:
                final_loss = float(line.split("loss:")[1].split("|")[0])
            except ValueError:
                pass
            break
    world = dist.get_world_size() if dist.is_initialized() else 1
    tokens_per_step = rows * seq * micro_steps * dp_world
    result = {
        "impl": "reference",
        "value": tokens_per_step / (ms_device / 1e3),
        "ms_per_step": ms_device,
        "e2e_value": tokens_per_step / (ms_e2e / 1e3),
        "e2e_ms_per_step": ms_e2e,
        "tokens_per_step": tokens_per_step,
        "h2d_bytes_per_step": 2 * rows * seq * 8 * micro_steps,
        "d2h_bytes_per_step": 4,
        "clocks": clocks,
        "loss": final_loss,
        "parallelism": compositions.describe(spec, world),
        "composition": composition,
        "is_rank0": engine.is_global_zero,
    }
    engine.close()
    return result
