"""One training script for every model under ``experiments/`` (the reference carries a ~300-line
``train.py`` per folder that differs in the model it builds: experiments/template/train.py,
experiments/griffin_and_hawk/train_gnh.py, experiments/mHC/train.py, ...).

    python experiments/train_experiment.py --model griffin --steps 200
    python experiments/train_experiment.py --model mhc --text my_corpus.txt --device cuda

Byte-level language modelling on ``--text`` (any file; without it a synthetic corpus with
repeating structure, so that the loss has something to learn), AdamW with warm-up and cosine decay,
bf16 autocast on CUDA. Prints the loss every ``--log-every`` steps and a final JSON line with the
first and last smoothed loss, parameters and tokens per second. Models: ``mqa`` / ``hawk`` /
``griffin``; ``residual`` / ``hc`` / ``mhc``; the template variants ``baseline`` / ``kattention`` /
``partial_kv`` / ``xglu`` / ``deglu`` / ``springnet`` / ``tokenformer`` / ``tokenformer_full`` /
``mla`` / ``relu2`` / ``mixture_of_depth`` / ``hypersphere`` / ``bitnet``; ``life`` trains the
template baseline on Game of Life transitions with the loss on the next board only."""

from __future__ import annotations

import argparse
import json
import math
import sys
import time
from pathlib import Path

import torch
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

RECURRENT = ("mqa", "hawk", "griffin")
CONNECTIONS = ("residual", "hc", "mhc")


def build_model(name: str, vocab: int, args) -> torch.nn.Module:
    if name in RECURRENT:
        from experiments.griffin_and_hawk.model import HawkAndGriffin, HnGConfig

        return HawkAndGriffin(HnGConfig(model_type=name, vocab_size=vocab, seq_len=args.seq_len,
                                        dim=args.dim, num_heads=args.heads, num_kv_heads=1,
                                        num_layers=args.layers))
    if name in CONNECTIONS:
        from experiments.mhc.model import MHCConfig, MHCModel

        return MHCModel(MHCConfig(vocab_size=vocab, max_sequence_length=args.seq_len,
                                  hidden_size=args.dim, intermediate_size=args.dim * 8 // 3,
                                  num_attention_heads=args.heads, num_hidden_layers=args.layers,
                                  connection_type=name))
    from experiments.template.model import TemplateConfig, build

    cfg = TemplateConfig(vocab_size=vocab, seq_len=args.seq_len, d_model=args.dim,
                         hidden_dim=args.dim * 8 // 3 // 4 * 4, num_heads=args.heads,
                         num_layers=args.layers)
    return build("baseline" if name == "life" else name, cfg)


def synthetic_corpus(length: int, seed: int = 0) -> torch.Tensor:
    """Bytes with structure at several scales: a small vocabulary of random "words" drawn from a
    first-order Markov chain."""
    generator = torch.Generator().manual_seed(seed)
    words = [torch.randint(97, 123, (int(n),), generator=generator)
             for n in torch.randint(2, 8, (64,), generator=generator)]
    transition = torch.rand(64, 64, generator=generator).pow(8)
    out, current, total = [], 0, 0
    while total < length:
        current = int(torch.multinomial(transition[current], 1, generator=generator))
        out += [words[current], torch.tensor([32])]
        total += len(words[current]) + 1
    return torch.cat(out)[:length]


def text_batches(data: torch.Tensor, batch: int, seq_len: int, generator: torch.Generator):
    while True:
        starts = torch.randint(0, data.numel() - seq_len - 1, (batch,), generator=generator)
        rows = torch.stack([data[s : s + seq_len + 1] for s in starts.tolist()])
        yield rows[:, :-1], rows[:, 1:], None


def life_batches(batch: int, size: int, seed: int):
    from experiments.lifelm.life import LifeDataset, boards_to_tokens

    stream = iter(LifeDataset(size, 10**9, seed=seed))
    while True:
        pairs = [next(stream) for _ in range(batch)]
        tokens, mask = boards_to_tokens(torch.stack([a for a, _ in pairs]),
                                        torch.stack([b for _, b in pairs]))
        yield tokens[:, :-1], tokens[:, 1:], mask[:, 1:]


def main(argv=None) -> dict:
    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default="griffin")
    parser.add_argument("--text", default=None)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--batch", type=int, default=16)
    parser.add_argument("--seq-len", type=int, default=128)
    parser.add_argument("--dim", type=int, default=128)
    parser.add_argument("--heads", type=int, default=4)
    parser.add_argument("--layers", type=int, default=4)
    parser.add_argument("--lr", type=float, default=3e-3)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--weight-decay", type=float, default=0.1)
    parser.add_argument("--aux-weight", type=float, default=0.01)
    parser.add_argument("--life-size", type=int, default=8)
    parser.add_argument("--log-every", type=int, default=50)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = parser.parse_args(argv)
    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    generator = torch.Generator().manual_seed(args.seed)
    if args.model == "life":
        from experiments.lifelm.life import VOCAB_SIZE

        vocab = VOCAB_SIZE
        args.seq_len = 2 * args.life_size**2
        batches = life_batches(args.batch, args.life_size, args.seed)
    else:
        vocab = 256
        data = (torch.tensor(list(Path(args.text).read_bytes()), dtype=torch.long) if args.text
                else synthetic_corpus(200_000, args.seed))
        batches = text_batches(data, args.batch, args.seq_len, generator)
    model = build_model(args.model, vocab, args).to(device)
    decay = [p for p in model.parameters() if p.ndim >= 2]
    rest = [p for p in model.parameters() if p.ndim < 2]
    optimizer = torch.optim.AdamW([{"params": decay, "weight_decay": args.weight_decay},
                                   {"params": rest, "weight_decay": 0.0}], lr=args.lr,
                                  betas=(0.9, 0.95))

    def rate(step: int) -> float:
        if step < args.warmup:
            return args.lr * (step + 1) / args.warmup
        progress = (step - args.warmup) / max(1, args.steps - args.warmup)
        return args.lr * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * progress)))

    losses, began = [], time.perf_counter()
    for step in range(args.steps):
        inputs, targets, mask = next(batches)
        inputs, targets = inputs.to(device), targets.to(device)
        for group in optimizer.param_groups:
            group["lr"] = rate(step)
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=device.type == "cuda"):
            logits = model(inputs)
        per_token = F.cross_entropy(logits.float().flatten(0, 1), targets.flatten(), reduction="none")
        if mask is not None:
            weights = mask.to(device).flatten().float()
            loss = (per_token * weights).sum() / weights.sum()
        else:
            loss = per_token.mean()
        total = loss
        extra = getattr(model, "auxiliary_loss", None)
        if extra is not None:
            total = total + args.aux_weight * extra
        optimizer.zero_grad(set_to_none=True)
        total.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        optimizer.step()
        losses.append(float(loss.detach()))
        if args.log_every and (step + 1) % args.log_every == 0:
            print(f"step {step + 1:5d} loss {sum(losses[-args.log_every:]) / args.log_every:.4f} "
                  f"lr {rate(step):.2e}", flush=True)
    elapsed = time.perf_counter() - began
    window = max(1, min(10, args.steps // 4))
    result = {
        "model": args.model,
        "parameters": sum(p.numel() for p in model.parameters()),
        "first_loss": sum(losses[:window]) / window,
        "last_loss": sum(losses[-window:]) / window,
        "tokens_per_second": args.steps * args.batch * args.seq_len / elapsed,
        "device": device.type,
    }
    print(json.dumps(result))
    return result


if __name__ == "__main__":
    main()
