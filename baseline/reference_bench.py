"""Reference arm of the headline benchmark.

Runs the *unmodified* reference package (``ohara``, installed from the read-only source tree into
``baseline/_ref`` with ``pip install --no-index --no-deps --target``) through its own public API:
``ohara.Llama`` / ``Config``, ``OharaEngine`` (single device, or its DDP strategy under torchrun),
``ohara.optimizer.build_muon_adamw`` and ``ohara.Trainer.train``. None of this package's models,
kernels or engine is imported here. The only addition is a stub ``lightning`` module that the
reference imports for a parameter summary and that is not installed on this image.

Timing: ``Trainer.train`` is called once for the warm-up iterations and once more (``start_iter``
= warm-up) for the timed iterations, bracketed by a barrier + ``torch.cuda.synchronize()`` and CUDA
events; the maximum over ranks is reported.
"""

from __future__ import annotations

import contextlib
import io
import os
import sys
from pathlib import Path


def reference_available() -> tuple[bool, str]:
    root = Path(__file__).resolve().parent / "_ref" / "ohara"
    if not root.is_dir():
        return False, "baseline/_ref/ohara is missing (reference not installed)"
    return True, ""


def run(args, model_cfg: dict, clock_sampler) -> dict:
    here = Path(__file__).resolve().parent
    sys.path.insert(0, str(here / "stubs"))
    sys.path.insert(0, str(here / "_ref"))
    import torch
    import torch.distributed as dist
    from torch.utils.data import DataLoader, IterableDataset

    from ohara import Config, Llama, OharaEngine, Trainer  # the reference package
    from ohara.lr_scheduler import Scheduler
    from ohara.optimizer import build_muon_adamw

    torch.manual_seed(1234 + int(os.environ.get("RANK", "0")))
    torch.set_float32_matmul_precision("high")  # as examples/train_llama_engine.py:226 does
    engine = OharaEngine()
    engine.launch()
    device = engine.device

    cfg = Config(
        vocab_size=model_cfg["vocab_size"], max_sequence_length=model_cfg["seq_len"],
        hidden_size=model_cfg["hidden_size"], intermediate_size=model_cfg["intermediate_size"],
        num_attention_heads=model_cfg["num_heads"], num_key_value_heads=0,
        num_hidden_layers=model_cfg["num_layers"], dropout=0.0, weight_tying=False,
        rope_theta=10000.0,
    )
    model = engine.prepare(Llama(cfg))
    optimizer = build_muon_adamw(model)

    batch, seq, vocab = model_cfg["batch_per_gpu"], model_cfg["seq_len"], model_cfg["vocab_size"]

    class Synthetic(IterableDataset):
        """Uniform random token rows generated on the host, one pinned batch per step."""

        def __iter__(self):
            gen = torch.Generator().manual_seed(99 + int(os.environ.get("RANK", "0")))
            while True:
                rows = torch.randint(0, vocab, (batch, seq + 1), generator=gen)
                yield rows[:, :-1].contiguous().pin_memory(), rows[:, 1:].contiguous().pin_memory()

    loader = DataLoader(Synthetic(), batch_size=None)
    train_dl, val_dl = engine.prepare_dataloaders(loader, loader)
    total = args.warmup + args.steps
    trainer = Trainer(
        engine, model, optimizer, train_dl, val_dl, Scheduler(0.02), micro_batch=1,
        max_iters=max(args.warmup, 1), eval_iters=0, save_ckpt_iters=0, print_every=10**9,
        flops_per_token=1.0, peak_flops=1.0,
    )

    def sync():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    quiet = io.StringIO()
    with contextlib.redirect_stdout(quiet):
        if args.warmup > 0:
            trainer.train(start_iter=0)
        trainer.max_iters = total
        sync()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clock_sampler.start()
        start.record()
        trainer.train(start_iter=args.warmup)
        stop.record()
        sync()
        clocks = clock_sampler.stop()
    elapsed_ms = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed_ms.item()) / args.steps
    world = dist.get_world_size() if dist.is_initialized() else 1
    tokens_per_step = batch * seq * world
    value = tokens_per_step / (ms_per_step / 1e3)
    result = {
        "impl": "reference",
        "value": value,
        "ms_per_step": ms_per_step,
        "tokens_per_step": tokens_per_step,
        "h2d_bytes_per_step": 2 * batch * seq * 8,
        "d2h_bytes_per_step": 4,
        "clocks": clocks,
        "parallelism": "single" if world == 1 else f"ddp{world}",
        "is_rank0": engine.is_global_zero,
    }
    engine.close()
    return result
