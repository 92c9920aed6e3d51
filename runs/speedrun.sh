#!/bin/bash
# Stage a corpus, pretrain a Llama on it, finetune it into a chat model and serve it.
#
#   bash runs/speedrun.sh
#   screen -L -Logfile runs/speedrun.log -S speedrun bash runs/speedrun.sh   # detachable
#
# DEPTH is the one size dial: width, batch size, learning rates, weight decay and the token
# horizon all come from the scaling planner. Environment overrides:
#   DEPTH (12)  NPROC (all visible GPUs)  DEVICE_BATCH_SIZE (32)  SEQ_LEN (2048)
#   TOKEN_RATIO tokens per effective parameter (12)  SHARDS ClimbMix shards to stage (24)
#   TRAIN_DOCS / VAL_DOCS  TOKENIZER  DATA_DIR  CKPT_DIR  SFT_ITERS (800)
#   NUM_WORKERS dataloader processes per rank (1; use 0 with --resume so that the stream position is exact)
#   STRATEGY multi-GPU strategy: fsdp = sharded optimizer over NVLink peer memory (default), ddp
#   SERVE start the chat UI at the end (1)  PORT (8080)
set -euo pipefail

DEPTH="${DEPTH:-12}"
SEQ_LEN="${SEQ_LEN:-2048}"
DEVICE_BATCH_SIZE="${DEVICE_BATCH_SIZE:-32}"
TOKEN_RATIO="${TOKEN_RATIO:-12}"
SHARDS="${SHARDS:-24}"
TRAIN_DOCS="${TRAIN_DOCS:-4000000}"
VAL_DOCS="${VAL_DOCS:-20000}"
TOKENIZER="${TOKENIZER:-EleutherAI/gpt-neo-125m}"
DATA_DIR="${DATA_DIR:-./data/scaling_corpus}"
CKPT_DIR="${CKPT_DIR:-./ckpt}"
STRATEGY="${STRATEGY:-fsdp}"
NUM_WORKERS="${NUM_WORKERS:-1}"
SERVE="${SERVE:-1}"
PORT="${PORT:-8080}"
SFT_ITERS="${SFT_ITERS:-800}"
export OMP_NUM_THREADS=1

cd "$(dirname "$0")/.."
if [ -z "${NPROC:-}" ]; then
  NPROC=$(python -c 'import torch; print(max(1, torch.cuda.device_count()))' 2>/dev/null || echo 1)
fi
RUN="d${DEPTH}"
BASE_CKPT="${CKPT_DIR}/base_${RUN}.pt"
SFT_CKPT="${CKPT_DIR}/sft_${RUN}.pt"
mkdir -p "$CKPT_DIR" runs

echo "== ohara_b200 speedrun: depth=${DEPTH} gpus=${NPROC} seq_len=${SEQ_LEN}" \
     "tokens/param=${TOKEN_RATIO} device_batch=${DEVICE_BATCH_SIZE} strategy=${STRATEGY}"

# 1) Data: stage text locally, then tokenise it once into memory-mapped token bins so the
#    training loop never tokenises and never touches the network.
if [ -f "${DATA_DIR}/train.jsonl" ]; then
  echo "[1/4] corpus already staged at ${DATA_DIR}, skipping"
else
  echo "[1/4] staging ClimbMix corpus -> ${DATA_DIR}"
  python examples/prepare_scaling_data.py --climbmix-train-shards "${SHARDS}" \
    --train-documents "${TRAIN_DOCS}" --validation-documents "${VAL_DOCS}" \
    --tokenizer "${TOKENIZER}" --output-dir "${DATA_DIR}" --skip-existing
fi
python examples/pretokenize_corpus.py --corpus "${DATA_DIR}" --tokenizer "${TOKENIZER}" --chat-tokens

# 2) Plan: every hyperparameter from DEPTH. The chat tokens are counted so that the planned
#    vocabulary is the one pretraining builds.
echo "[2/4] planning depth=${DEPTH}"
eval "$(python - <<PY
from ohara_b200.chat import CHAT_SPECIAL_TOKENS
from ohara_b200.scaling import plan_scaling_run
from ohara_b200.tokenizer import get_tokenizer

vocab = len(get_tokenizer(hf_name="${TOKENIZER}", prefer_hf=True)) + len(CHAT_SPECIAL_TOKENS)
plan = plan_scaling_run(${DEPTH}, vocab_size=vocab, target_param_data_ratio=${TOKEN_RATIO},
                        sequence_length=${SEQ_LEN}, device_batch_size=${DEVICE_BATCH_SIZE},
                        world_size=${NPROC})
names = {"HIDDEN_SIZE": "hidden_size", "INTERMEDIATE_SIZE": "intermediate_size",
         "NUM_HEADS": "num_heads", "GRAD_ACCUM": "grad_accum_steps", "MAX_ITERS": "num_iterations",
         "MATRIX_LR": "matrix_learning_rate", "EMBEDDING_LR": "embedding_learning_rate",
         "UNEMBEDDING_LR": "unembedding_learning_rate", "SCALAR_LR": "scalar_learning_rate",
         "WEIGHT_DECAY": "weight_decay", "PARAMS_EFFECTIVE": "params_effective",
         "TOKENS_TRAINED": "tokens_trained", "TOTAL_BATCH_SIZE": "total_batch_size"}
for shell_name, field in names.items():
    print(f"{shell_name}={getattr(plan, field)}")
PY
)"
printf ' model:  %s effective params, hidden=%s ffn=%s heads=%s\n' \
  "$PARAMS_EFFECTIVE" "$HIDDEN_SIZE" "$INTERMEDIATE_SIZE" "$NUM_HEADS"
printf ' budget: %s tokens over %s iters, batch %s tokens (accum %s)\n' \
  "$TOKENS_TRAINED" "$MAX_ITERS" "$TOTAL_BATCH_SIZE" "$GRAD_ACCUM"

# 3) Pretrain.
if [ "$NPROC" -gt 1 ]; then
  LAUNCH="python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=${NPROC}"
else
  LAUNCH="python"
  STRATEGY="auto"
fi
echo "[3/4] pretraining -> ${BASE_CKPT}"
$LAUNCH examples/train_llama_engine.py \
  --dataset "${DATA_DIR}" --tokenizer "${TOKENIZER}" --chat-tokens --pad-vocab-to 128 \
  --seq-len "${SEQ_LEN}" --batch-size "${DEVICE_BATCH_SIZE}" --grad-accum-steps "${GRAD_ACCUM}" \
  --max-iters "${MAX_ITERS}" --hidden-size "${HIDDEN_SIZE}" \
  --intermediate-size "${INTERMEDIATE_SIZE}" --num-layers "${DEPTH}" --num-heads "${NUM_HEADS}" \
  --optimizer muon --init-style nanochat --no-weight-tying --lr-schedule wsd \
  --matrix-learning-rate "${MATRIX_LR}" --embedding-learning-rate "${EMBEDDING_LR}" \
  --unembedding-learning-rate "${UNEMBEDDING_LR}" --scalar-learning-rate "${SCALAR_LR}" \
  --weight-decay "${WEIGHT_DECAY}" --evaluate-bpb --strategy "${STRATEGY}" \
  --num-workers "${NUM_WORKERS}" \
  --eval-every 250 --save-every 500 --checkpoint-path "${BASE_CKPT}" \
  --result-json "runs/base_${RUN}.json"

# 4) Finetune: teaches the conversation format; minutes next to pretraining.
echo "[4/4] supervised finetuning -> ${SFT_CKPT}"
$LAUNCH examples/train_sft.py \
  --pretrained-checkpoint "${BASE_CKPT}" --checkpoint-path "${SFT_CKPT}" \
  --tokenizer "${TOKENIZER}" --seq-len "${SEQ_LEN}" --batch-size "${DEVICE_BATCH_SIZE}" \
  --grad-accum-steps "${GRAD_ACCUM}" --max-iters "${SFT_ITERS}" \
  --num-workers "${NUM_WORKERS}" \
  --result-json "runs/sft_${RUN}.json"

echo
echo "done. base=${BASE_CKPT} sft=${SFT_CKPT}"
if [ "$SERVE" = "1" ]; then
  echo "starting chat UI on port ${PORT} (from a laptop: ssh -N -L ${PORT}:localhost:${PORT} <user>@<host>)"
  python examples/chat_web.py --checkpoint "${SFT_CKPT}" --port "${PORT}"
else
  echo "chat with it:  python examples/chat_web.py --checkpoint ${SFT_CKPT}"
fi
