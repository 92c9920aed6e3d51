#!/bin/bash
# Run every benchmark configuration of bench.py, both arms, at 1 / 2 / 4 / 8 GPUs of one node, plus
# the decoding, kernel and CPU benchmarks, and collect the JSON lines.
#
#   bash runs/benchmarks.sh                      # everything the visible GPUs allow
#   CONFIGS="d12 moe_ep8" GPUS="1 8" bash runs/benchmarks.sh
#
# Environment overrides:
#   OUT      output folder (./runs/benchmarks)
#   CONFIGS  configurations of bench.py ("d12 sft_d12 tp4_fsdp2_1p3b cp8_32k moe_ep8 moe_ep8_skewed
#            fsdp_1p3b fsdp_1p3b_sharded_parameters")
#   GPUS     GPU counts to run ("1 2 4 8", capped at the visible devices)
#   ARMS     "ours reference" (the reference arm needs the reference package under baseline/_ref)
#   STEPS / WARMUP  timed and untimed steps per run (4 / 3)
#   PORT     first rendezvous port (29500)
# Every run writes OUT/<config>_n<gpus>_<arm>.json (the one JSON line of bench.py) and a log beside
# it; a failed run leaves only its log and the script goes on. All timing is done by bench.py on the
# device (CUDA events, maximum over ranks); nothing here changes any GPU setting.
set -uo pipefail

cd "$(dirname "$0")/.."
OUT="${OUT:-./runs/benchmarks}"
CONFIGS="${CONFIGS:-d12 sft_d12 tp4_fsdp2_1p3b cp8_32k moe_ep8 moe_ep8_skewed fsdp_1p3b fsdp_1p3b_sharded_parameters}"
GPUS="${GPUS:-1 2 4 8}"
ARMS="${ARMS:-ours reference}"
STEPS="${STEPS:-4}"
WARMUP="${WARMUP:-3}"
PORT="${PORT:-29500}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-1}"
mkdir -p "$OUT"

VISIBLE=$(python -c 'import torch; print(torch.cuda.device_count())' 2>/dev/null || echo 0)
echo "visible GPUs: ${VISIBLE}; results in ${OUT}"

run_bench() {  # config gpus arm
  local config="$1" gpus="$2" arm="$3"
  local stem="${OUT}/${config}_n${gpus}_${arm}"
  local flags=(--config "$config" --gpus "$gpus" --steps "$STEPS" --warmup "$WARMUP")
  if [ "$arm" = "reference" ]; then flags+=(--impl reference); fi
  PORT=$((PORT + 1))
  if [ "$gpus" -gt 1 ]; then
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$gpus" --master-addr 127.0.0.1 \
      --master-port "$PORT" bench.py "${flags[@]}" > "${stem}.log" 2>&1
  else
    python bench.py "${flags[@]}" > "${stem}.log" 2>&1
  fi
  local code=$?
  if [ "$code" -eq 0 ] && grep -q '^{' "${stem}.log"; then
    grep '^{' "${stem}.log" | tail -n 1 > "${stem}.json"
    python - "$stem.json" <<'PY'
import json, sys
line = json.load(open(sys.argv[1]))
if "unavailable" in line:
    print(f"  {sys.argv[1]}: unavailable ({line['unavailable']})")
else:
    print(f"  {sys.argv[1]}: {line['value']:,.0f} {line['unit']}, {line['ms_per_step']:.1f} ms/step")
PY
  else
    echo "  ${stem}: failed (exit ${code}), see ${stem}.log"
  fi
}

if [ "$VISIBLE" -ge 1 ]; then
  for config in $CONFIGS; do
    for gpus in $GPUS; do
      if [ "$gpus" -gt "$VISIBLE" ]; then continue; fi
      for arm in $ARMS; do
        echo "bench ${config} on ${gpus} GPU(s), ${arm}"
        run_bench "$config" "$gpus" "$arm"
      done
    done
  done
  echo "decoding (batch 1 / 16 / 64)"
  python examples/bench_decode.py > "${OUT}/decode_n1.log" 2>&1 || echo "  failed, see ${OUT}/decode_n1.log"
  if [ "$VISIBLE" -ge 8 ]; then
    PORT=$((PORT + 1))
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port "$PORT" examples/bench_decode.py --tp 8 > "${OUT}/decode_tp8.log" 2>&1 \
      || echo "  failed, see ${OUT}/decode_tp8.log"
  fi
  echo "kernels against the libraries"
  python examples/bench_kernels.py > "${OUT}/kernels.log" 2>&1 || echo "  failed, see ${OUT}/kernels.log"
else
  echo "no GPU visible: GPU benchmarks skipped"
fi

echo "CPU configuration (tiny Llama, fp32)"
for arm in $ARMS; do
  python examples/bench_cpu_tiny_llama.py --impl "$arm" 2> /dev/null | grep '^{' > "${OUT}/cpu_tiny_llama_${arm}.json" \
    && cat "${OUT}/cpu_tiny_llama_${arm}.json"
done
