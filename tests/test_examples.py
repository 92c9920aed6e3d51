"""The example programs: finetuning checkpoint loader, safetensors export, status dashboard and a
short end-to-end pretraining run. (Reference suite for the loader: tests/test_train_sft.py:48-124.)"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import threading
import urllib.request
from pathlib import Path

import pytest
import torch

from helpers import chat_tokenizer, tiny_llama
from test_data import EXAMPLES, load_example


@pytest.fixture(scope="module")
def sft():
    return load_example("train_sft")


def save(model, path, prefix=""):
    torch.save({"model": {prefix + k: v for k, v in model.state_dict().items()}, "idx": 11}, path)
    return path


def test_loader_rebuilds_the_base_and_grows_the_vocabulary(sft, tmp_path):
    tok = chat_tokenizer()
    base = tiny_llama(len(tok) - 4, context=32, num_key_value_heads=1, weight_tying=False)
    path = save(base, tmp_path / "base.pt")
    model, config, old_vocab = sft.load_pretrained(path, len(tok), None)
    assert old_vocab == len(tok) - 4 and model.token_emb.weight.shape[0] == len(tok)
    assert config.num_key_value_heads == 1 and config.max_sequence_length == 32
    assert torch.equal(model.token_emb.weight[:old_vocab], base.token_emb.weight)
    assert torch.equal(model.layers[1].ff.down.weight, base.layers[1].ff.down.weight)
    wider, _, _ = sft.load_pretrained(save(tiny_llama(len(tok) + 16), tmp_path / "w.pt"), len(tok), None)
    assert wider.token_emb.weight.shape[0] == len(tok) + 16, "spare padded rows are kept"


def test_loader_keeps_tying_and_handles_context_and_prefixes(sft, tmp_path):
    tok = chat_tokenizer()
    tied = save(tiny_llama(len(tok) - 2, context=32, weight_tying=True), tmp_path / "tied.pt")
    model, _, _ = sft.load_pretrained(tied, len(tok), 16)
    assert model.vocab_proj.weight is model.token_emb.weight
    assert model.config.max_sequence_length == 16
    assert model(torch.randint(0, len(tok), (1, 16))).shape == (1, 16, len(tok))
    with pytest.raises(ValueError, match="exceeds the pretrained context"):
        sft.load_pretrained(tied, len(tok), 64)
    with pytest.raises(FileNotFoundError):
        sft.load_pretrained(tmp_path / "absent.pt", len(tok), None)
    wrapped = save(tiny_llama(len(tok)), tmp_path / "wrapped.pt", prefix="_orig_mod.module.")
    assert sft.load_pretrained(wrapped, len(tok), None)[1].vocab_size == len(tok)


def test_safetensors_export_round_trips(tmp_path):
    from safetensors.torch import load_file

    export = load_example("export_safetensors")
    model = tiny_llama(48, weight_tying=True, moe_num_experts=4, moe_experts_per_tok=2, moe_grouped=True)
    path = save(model, tmp_path / "moe.pt")
    summary = export.export(path, tmp_path / "out", moe_experts_per_tok=2)
    config = json.loads((tmp_path / "out" / "config.json").read_text())
    assert config["moe_num_experts"] == 4 and config["moe_grouped"] and config["iteration"] == 11
    tensors = load_file(tmp_path / "out" / "model.safetensors")
    assert summary["tensors"] == len(tensors)
    assert not any(name.endswith(export.DERIVED_BUFFERS) for name in tensors)
    assert torch.equal(tensors["token_emb.weight"], model.token_emb.weight)
    kept = export.export(path, tmp_path / "full", keep_derived_buffers=True)
    assert kept["tensors"] > summary["tensors"]


def test_status_dashboard_reads_a_multi_stage_log(tmp_path):
    status = load_example("train_status")
    log = tmp_path / "speedrun.log"
    log.write_text(
        "[3/4] pretraining -> ckpt/base.pt\n"
        " budget: 1,000,000 tokens over 40 iters, batch 1024 tokens (accum 1)\n"
        "device=cuda:0 precision=bf16_mixed params=1,234,567 tokens/step/rank=1,024\n"
        + "".join(f"iter: {i} | loss: {5 - i * 0.1:.4f} | lr: 1.0e-02 | time: 0.5000s | "
                  f"tok/s: 2,048.00 | mfu: 41.20% | eta: {(40 - i) * 0.5 / 60:.1f}m\n" for i in range(1, 11))
        + "iter: 10 | val_loss: 4.1000 | val_ppl: 60.3 | val_bits/token: 5.9 | val_acc: 0.2100 | "
          "val_bpb: 1.3100 | lr: 1.0e-02\n")
    state = status.parse_log(log)
    assert state["stage"].startswith("pretraining") and state["total_iters"] == 40
    assert state["iter"] == 10 and state["percent"] == 25.0 and state["params"] == 1_234_567
    assert state["median_step_seconds"] == 0.5 and state["remaining_minutes"] == 0.2
    assert state["tokens_per_sec"] == 2048 and state["mfu"] == 41.2 and len(state["history"]) == 10
    assert state["val"] == [{"iter": 10, "loss": 4.1, "acc": 0.21, "bpb": 1.31}]
    with open(log, "a") as handle:
        handle.write("[4/4] supervised finetuning -> ckpt/sft.pt\nbefore SFT: val_loss=4.0\n"
                     "iter: 1 | loss: 3.0000 | lr: 1.0e-02 | time: 0.2000s\nafter SFT: val_loss=2.0\n")
    state = status.parse_log(log, total_override=4)
    assert state["stage"].startswith("supervised") and state["finished"] and state["percent"] == 100.0
    assert len(state["history"]) == 1
    assert status.parse_log(tmp_path / "absent.log")["error"]

    server = status.create_server(log, "127.0.0.1", 0)
    thread = threading.Thread(target=server.serve_forever, daemon=True)
    thread.start()
    try:
        base = f"http://127.0.0.1:{server.server_address[1]}"
        with urllib.request.urlopen(base + "/api/status", timeout=10) as reply:
            assert json.loads(reply.read())["finished"] is True
        with urllib.request.urlopen(base + "/", timeout=10) as reply:
            assert b"ohara_b200" in reply.read()
    finally:
        server.shutdown()
        server.server_close()
        thread.join(timeout=5)


def test_pretraining_example_trains_saves_and_resumes(tmp_path):
    checkpoint, result = tmp_path / "ckpt" / "model.pt", tmp_path / "result.json"
    command = [sys.executable, str(EXAMPLES / "train_llama_engine.py"), "--synthetic",
               "--synthetic-vocab", "256", "--seq-len", "32", "--hidden-size", "32",
               "--intermediate-size", "64", "--num-layers", "2", "--num-heads", "2",
               "--batch-size", "2", "--grad-accum-steps", "2", "--warmup-iters", "1",
               "--eval-every", "2", "--eval-batches", "1", "--save-every", "2", "--logger", "none",
               "--precision", "fp32", "--no-weight-tying", "--checkpoint-path", str(checkpoint),
               "--result-json", str(result)]
    first = subprocess.run(command + ["--max-iters", "2"], capture_output=True, text=True, timeout=300)
    assert first.returncode == 0, first.stderr[-2000:]
    assert checkpoint.exists() and "final val_loss=" in first.stdout
    report = json.loads(result.read_text())
    assert report["num_iterations"] == 2 and report["total_batch_size"] == 2 * 32 * 2
    assert report["params_total"] == report["params_effective"] + report["params_token_embeddings"] \
        + report["params_norms_and_scalars"]
    second = subprocess.run(command + ["--max-iters", "4", "--resume"], capture_output=True,
                            text=True, timeout=300)
    assert second.returncode == 0, second.stderr[-2000:]
    assert "resumed checkpoint" in second.stdout and "iter: 3 |" in second.stdout
    assert "iter: 1 |" not in second.stdout


@pytest.mark.parametrize("layout", [
    ["--strategy", "ddp"],
    ["--strategy", "fsdp", "--pp", "2", "--optimizer", "adamw"],
])
def test_pretraining_example_on_two_ranks_saves_and_resumes(tmp_path, layout):
    """The same script under torchrun on two CPU ranks: plain DDP (whose wrapper must take the
    wrapper-free checkpoint back) and two pipeline stages (whose checkpoint is the whole
    model)."""
    checkpoint = tmp_path / "ckpt" / "model.pt"
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", str(32500 + os.getpid() % 300),
               str(EXAMPLES / "train_llama_engine.py"), "--synthetic", "--synthetic-vocab", "256",
               "--seq-len", "32", "--hidden-size", "32", "--intermediate-size", "64",
               "--num-layers", "2", "--num-heads", "2", "--batch-size", "2",
               "--grad-accum-steps", "2", "--warmup-iters", "1", "--eval-every", "2",
               "--eval-batches", "1", "--save-every", "2", "--logger", "none", "--precision", "fp32",
               "--no-weight-tying", "--checkpoint-path", str(checkpoint), *layout]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    first = subprocess.run(command + ["--max-iters", "2"], capture_output=True, text=True,
                           timeout=300, env=env)
    assert first.returncode == 0, first.stdout[-1500:] + first.stderr[-2500:]
    assert checkpoint.exists() and "final val_loss=" in first.stdout
    second = subprocess.run(command + ["--max-iters", "4", "--resume"], capture_output=True,
                            text=True, timeout=300, env=env)
    assert second.returncode == 0, second.stdout[-1500:] + second.stderr[-2500:]
    assert "resumed checkpoint" in second.stdout and "iter: 4 |" in second.stdout
    assert "iter: 1 |" not in second.stdout
    saved = torch.load(checkpoint, weights_only=False)
    assert saved["model"]["layers.1.attn.query.weight"].shape == (32, 32)   # whole matrices


def test_finetuning_example_runs_from_a_pretrained_checkpoint_to_a_chat_reply(tmp_path):
    """pretrain (synthetic ids) -> train_sft.py on a local JSONL with a local tokenizer -> the
    checkpoint and the tokenizer saved beside it answer through ChatEngine."""
    import random

    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast

    rng = random.Random(0)
    words = [f"w{i}" for i in range(60)] + "what is plus answer".split() + [str(i) for i in range(19)]
    corpus = [" ".join(rng.choice(words) for _ in range(20)) for _ in range(300)]
    raw = Tokenizer(models.BPE(unk_token="<unk>"))
    raw.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    raw.decoder = decoders.ByteLevel()
    raw.train_from_iterator(corpus, trainers.BpeTrainer(
        vocab_size=320, special_tokens=["<unk>", "<|endoftext|>"],
        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    PreTrainedTokenizerFast(tokenizer_object=raw, unk_token="<unk>", eos_token="<|endoftext|>",
                            bos_token="<|endoftext|>").save_pretrained(tmp_path / "tok")
    with open(tmp_path / "conversations.jsonl", "w") as handle:
        for _ in range(80):
            a, b = rng.randint(0, 9), rng.randint(0, 9)
            handle.write(json.dumps({"messages": [
                {"role": "user", "content": f"what is {a} plus {b}"},
                {"role": "assistant", "content": f"answer {a + b}"}]}) + "\n")

    base, tuned = tmp_path / "base.pt", tmp_path / "ckpt" / "sft.pt"
    pretrain = [sys.executable, str(EXAMPLES / "train_llama_engine.py"), "--synthetic",
                "--synthetic-vocab", "320", "--seq-len", "48", "--hidden-size", "32",
                "--intermediate-size", "64", "--num-layers", "2", "--num-heads", "2",
                "--batch-size", "2", "--max-iters", "2", "--warmup-iters", "1", "--eval-every", "0",
                "--save-every", "2", "--logger", "none", "--precision", "fp32",
                "--checkpoint-path", str(base)]
    done = subprocess.run(pretrain, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and base.exists(), done.stderr[-2000:]
    finetune = [sys.executable, str(EXAMPLES / "train_sft.py"), "--pretrained-checkpoint", str(base),
                "--checkpoint-path", str(tuned), "--tokenizer", str(tmp_path / "tok"),
                "--tokenizer-local-files-only", "--conversations",
                str(tmp_path / "conversations.jsonl"), "--seq-len", "48", "--batch-size", "4",
                "--max-iters", "6", "--eval-every", "3", "--eval-batches", "1", "--save-every", "6",
                "--logger", "none", "--precision", "fp32",
                "--result-json", str(tmp_path / "sft.json")]
    done = subprocess.run(finetune, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-1500:] + done.stderr[-2500:]
    assert "after SFT: val_loss=" in done.stdout and tuned.exists()
    assert (tuned.parent / "sft" / "ohara_chat.json").exists()

    bad = tmp_path / "bad.jsonl"
    bad.write_text(json.dumps([{"role": "user", "content": "hi"}]) + "\n")
    refused = subprocess.run(finetune[:finetune.index("--conversations") + 1] + [str(bad)]
                             + finetune[finetune.index("--conversations") + 2:],
                             capture_output=True, text=True, timeout=300)
    assert refused.returncode != 0 and "'messages'" in refused.stderr

    from ohara_b200.chat_engine import ChatEngine, SamplingConfig

    engine = ChatEngine.from_checkpoint(tuned, device="cpu")
    assert engine.model.config.vocab_size >= 320 + 6        # the chat tokens were added
    reply = engine.generate([{"role": "user", "content": "what is 2 plus 3"}],
                            SamplingConfig(temperature=0.0, max_new_tokens=4))
    assert isinstance(reply, str)


def test_sharded_run_of_two_ranks_resumes_on_one_rank_from_the_command_line(tmp_path):
    """Elastic restart: a run under the sharded optimizer saved by two ranks continues on one
    (the optimizer state is resharded on load, the data stream skips what was consumed)."""
    checkpoint = tmp_path / "ckpt" / "model.pt"
    script = [str(EXAMPLES / "train_llama_engine.py"), "--synthetic", "--synthetic-vocab", "256",
              "--seq-len", "32", "--hidden-size", "32", "--intermediate-size", "64",
              "--num-layers", "2", "--num-heads", "2", "--batch-size", "2", "--warmup-iters", "1",
              "--eval-every", "0", "--save-every", "2", "--logger", "none", "--precision", "fp32",
              "--strategy", "fsdp", "--checkpoint-path", str(checkpoint)]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    launcher = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                "--master-addr", "127.0.0.1", "--master-port", str(29650 + os.getpid() % 40)]
    first = subprocess.run(launcher + script + ["--max-iters", "2"], env=env, capture_output=True,
                           text=True, timeout=300)
    assert first.returncode == 0 and checkpoint.exists(), first.stderr[-2000:]
    second = subprocess.run([sys.executable] + script + ["--max-iters", "4", "--resume"], env=env,
                            capture_output=True, text=True, timeout=300)
    assert second.returncode == 0, second.stderr[-2000:]
    assert "resumed checkpoint" in second.stdout and "at iter=2" in second.stdout
    assert "iter: 4 |" in second.stdout and "iter: 1 |" not in second.stdout
