"""``bench.py --tiny``: every configuration's plumbing (model, parallel layout, optimizer, data,
both timing paths, the JSON line) at toy sizes on CPU. No benchmark number is checked."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _bench(*flags, world=1, env=None, port=29700):
    base = [sys.executable]
    if world > 1:
        base += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                 "--master-addr", "127.0.0.1", "--master-port", str(port + os.getpid() % 200)]
    cmd = base + [str(ROOT / "bench.py"), "--tiny", "--steps", "2", "--warmup", "1",
                  "--gpus", str(world), *flags]
    full_env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", **(env or {}))
    proc = subprocess.run(cmd, env=full_env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    lines = [line for line in proc.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, proc.stdout[-2000:]
    return json.loads(lines[0])


def test_resolve_names_the_layout_of_every_configuration():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.resolve("d12", 8, False)["parallelism"] == "fsdp8"
    tp = bench.resolve("tp4_fsdp2_1p3b", 8, False)
    assert (tp["tp"], tp["dp"], tp["parallelism"]) == (4, 2, "tp4 x fsdp2")
    assert tp["rows"] * tp["micro_steps"] * tp["dp"] == 256          # global batch of the config
    cp = bench.resolve("cp8_32k", 8, False)
    assert (cp["cp"], cp["dp"], cp["seq_len"], cp["parallelism"]) == (8, 1, 32768, "cp8")
    moe = bench.resolve("moe_ep8", 8, False)
    assert (moe["ep"], moe["dp"], moe["parallelism"]) == (8, 1, "ep8")
    assert bench.resolve("moe_ep8", 1, False)["parallelism"] == "single"
    assert bench.resolve("tp4_fsdp2_1p3b", 2, False)["tp"] == 2


@pytest.mark.parametrize("config", ["d12", "sft_d12", "moe_ep8_skewed", "cp8_32k"])
def test_tiny_configurations_run_on_one_process(config):
    line = _bench("--config", config)
    assert line["tiny"] is True and line["config"]["name"] == config
    assert line["value"] > 0 and line["e2e"]["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] > 0
    assert 3.0 < line["final_loss"] < 8.0
    if config == "sft_d12":
        assert 0 < line["supervised_tokens_per_batch"] < 4 * 128   # assistant tokens only


def test_tiny_tensor_parallel_times_sharded_optimizer_on_four_ranks():
    line = _bench("--config", "tp4_fsdp2_1p3b", world=4, env={"OHARA_BENCH_TP": "2"})
    assert line["config"]["parallelism"] == "tp2 x fsdp2"
    assert 3.0 < line["final_loss"] < 8.0


@pytest.mark.skipif(not (ROOT / "baseline" / "_ref" / "ohara").is_dir(),
                    reason="reference package is not installed")
def test_tiny_reference_arms_run():
    line = _bench("--impl", "reference", "--config", "sft_d12")
    assert line["impl"] == "reference" and line["config"]["composition"] == "reference as shipped"
    assert 3.0 < line["final_loss"] < 8.0
    line = _bench("--impl", "reference", "--config", "tp4_fsdp2_1p3b", world=4,
                  env={"OHARA_BENCH_TP": "2"}, port=30300)
    assert line["config"]["parallelism"] == "tp2 (DTensor) x fully_shard2"
    line = _bench("--impl", "reference", "--config", "moe_ep8", world=2, port=30900)
    assert line["config"]["parallelism"].startswith("ep2")


def test_tiny_data_parallel_config_with_sharded_parameters_on_two_ranks():
    plain = _bench("--config", "fsdp_1p3b", world=2, port=31500)
    sharded = _bench("--config", "fsdp_1p3b_sharded_parameters", world=2, port=32100)
    assert plain["config"]["parallelism"] == sharded["config"]["parallelism"] == "fsdp2"
    assert "parameter_memory" not in plain
    memory = sharded["parameter_memory"]
    assert memory["persistent_bytes_per_rank"] < 0.75 * memory["unsharded_bytes"]
    assert 0 < memory["peak_gathered_bytes"] < memory["unsharded_bytes"]
    # the same data, model and optimizer: both arrive at the same loss
    assert abs(plain["final_loss"] - sharded["final_loss"]) < 2e-3 * plain["final_loss"]


def test_tiny_context_parallel_configuration_on_two_ranks():
    line = _bench("--config", "cp8_32k", world=2, port=33300)
    assert line["config"]["parallelism"] == "cp2" and 3.0 < line["final_loss"] < 8.0


def test_tiny_expert_parallel_configuration_on_two_ranks():
    line = _bench("--config", "moe_ep8_skewed", world=2, port=32700)
    assert line["config"]["parallelism"] == "ep2"
    assert line["skew"]["target_share"] == 0.5 and 3.0 < line["final_loss"] < 8.0
    assert line["expert_load"]["dropped_pair_fraction_last_step"] > 0.0   # the skew overflows


def test_cpu_configuration_of_the_benchmark_set_reports_the_known_losses():
    """The tiny fp32 Llama of the benchmark set: its first loss is fixed by the seed (the value
    the reference package gives for the same loop)."""
    proc = subprocess.run([sys.executable, str(ROOT / "examples" / "bench_cpu_tiny_llama.py"),
                           "--steps", "4", "--threads", "2"], capture_output=True, text=True,
                          timeout=300, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads([row for row in proc.stdout.splitlines() if row.startswith("{")][-1])
    assert line["impl"] == "ours" and line["device"] == "cpu" and line["value"] > 0
    assert line["first_loss"] == pytest.approx(9.065635, abs=2e-5)
    assert line["last_loss"] < line["first_loss"] + 0.05
