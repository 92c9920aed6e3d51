"""Tensor-parallel decoding on two GPUs: the sharded model, whose row-parallel layers end in the
one-shot peer-memory all-reduce, must generate the tokens of the unsharded model, with and without
CUDA-graph replay of the decode step."""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_generation_matches_single_device(tmp_path):
    script = """
        import torch, torch.distributed as dist
        from ohara_b200 import ops
        from ohara_b200.chat import CHAT_SPECIAL_TOKENS
        from ohara_b200.chat_engine import ChatEngine, SamplingConfig
        from ohara_b200.models.llama import Config, Llama
        from ohara_b200.runtime import EngineConfig, OharaEngine, ParallelConfig, TensorParallelPlan

        class Vocabulary:
            eos_token_id = bos_token_id = pad_token_id = 0
            def __len__(self): return 512
            def get_vocab(self): return {t: 511 - i for i, t in enumerate(CHAT_SPECIAL_TOKENS)}

        torch.manual_seed(0)
        cfg = Config(vocab_size=512, max_sequence_length=128, hidden_size=256, intermediate_size=512,
                     num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, dropout=0.0)
        reference = Llama(cfg)
        state = {k: v.clone() for k, v in reference.state_dict().items()}
        engine = OharaEngine(EngineConfig(parallel=ParallelConfig(tp=2),
                                          tensor_parallel=TensorParallelPlan.llama_default(2)))
        engine.launch()
        prompt = torch.randint(1, 500, (3, 17), device=engine.device)
        solo = ChatEngine(reference, Vocabulary(), device=engine.device, dtype=torch.bfloat16)
        greedy = SamplingConfig(temperature=0.0, top_p=1.0, top_k=0, max_new_tokens=24)
        expected = solo.generate_batch(prompt, greedy, seed=1, cuda_graph=False)

        model = Llama(cfg)
        model.load_state_dict(state)
        model = engine.prepare_module(model.to(torch.bfloat16))
        row_parallel = [m for m in model.modules() if type(m).__name__ == "RowParallelLinear"]
        assert row_parallel and all(m.peer_runtime is not None for m in row_parallel)
        sharded = ChatEngine(model, Vocabulary(), device=engine.device, dtype=torch.bfloat16)
        launches = ops.ext().launch_count()
        eager = sharded.generate_batch(prompt, greedy, seed=1, cuda_graph=False)
        assert ops.ext().launch_count() > launches
        replay = sharded.generate_batch(prompt, greedy, seed=1, cuda_graph=True)
        again = sharded.generate_batch(prompt, greedy, seed=1, cuda_graph=True)
        torch.cuda.synchronize()
        ops.check_status()
        # bf16 sums in a different order can flip a near-tie: require agreement, not identity
        agree = (eager == expected).float().mean().item()
        assert agree > 0.9, agree
        assert torch.equal(replay, eager) and torch.equal(again, eager)
        # every rank must have generated exactly the same tokens
        gathered = [torch.empty_like(eager) for _ in range(2)]
        dist.all_gather(gathered, eager)
        assert torch.equal(gathered[0], gathered[1])
        if dist.get_rank() == 0:
            print("TP_DECODE_OK", agree)
        engine.close()
    """
    path = tmp_path / "worker.py"
    path.write_text(textwrap.dedent(script))
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29800 + os.getpid() % 90), str(path)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "TP_DECODE_OK" in proc.stdout
