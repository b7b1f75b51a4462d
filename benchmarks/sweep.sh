#!/bin/bash
# Sequence-length sweep of the four parallel modes on one node, the layout of the reference's published tables
# (reference README.md:39-45, run.sh:1-38): Llama-2-7B, bf16, batch 1, no activation checkpointing, AdamW every step.
#
#   GPU_NUM=8 SEQLENS="32768 65536 131072" MODES="odysseus tpsp ulysses ring" OUT=sweep.jsonl benchmarks/sweep.sh
#
# Every run appends its per-step records and a final record (tokens/s from max-over-ranks device time, peak GB,
# exposed communication ms) to $OUT; a run that does not fit prints "OOM", as the reference's tables do.
# HYBRID=1 adds Llama-3-8B at 256K on the Odysseus x ring and Ulysses x ring hybrids (inner degree 4, ring degree 2,
# activation checkpointing on: 32K tokens per GPU do not fit otherwise; HYBRID_L / HYBRID_U / HYBRID_R change the sequence
# length and the two degrees, e.g. 131072 on 2 x 2 GPUs).  EXTRA holds further train.py flags for the
# sweep runs, e.g. EXTRA="--grad-checkpoint" where the tokens per GPU need it.
GPU_NUM=${GPU_NUM:-8}
SEQLENS=${SEQLENS:-"32768 65536 131072"}
MODES=${MODES:-"odysseus tpsp ulysses ring"}
MODEL=${MODEL:-llama2-7b}
BACKEND=${BACKEND:-fused}
STEPS=${STEPS:-6}
WARMUP=${WARMUP:-2}
OUT=${OUT:-sweep.jsonl}
PORT=${PORT:-29540}
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
cd "$(dirname "$0")/.."

run() {   # mode seqlen extra-args...
  local mode=$1 L=$2; shift 2
  local log
  log=$(mktemp)
  python -m torch.distributed.run --nnodes=1 --nproc-per-node=$GPU_NUM --master-addr 127.0.0.1 --master-port $PORT \
    train.py --model-config $MODEL --seq-length $L --parallel_mode $mode --backend $BACKEND \
    --max-train-steps $STEPS --warmup-iterations $WARMUP --jsonl $OUT "$@" > $log 2>&1
  local rc=$?
  if grep -q "out of memory\|OutOfMemoryError" $log; then
    echo "{\"final\": true, \"mode\": \"$mode\", \"seq_length\": $L, \"world\": $GPU_NUM, \"model\": \"$MODEL\", \"result\": \"OOM\"}" >> $OUT
    echo "$MODEL $mode $((L/1024))K $GPU_NUM: OOM"
  elif [ $rc -ne 0 ]; then
    echo "$MODEL $mode $((L/1024))K $GPU_NUM: failed (rc $rc)"; tail -5 $log
  else
    grep -E "Time taken|device time" $log
  fi
  rm -f $log
}

for L in $SEQLENS; do
  for mode in $MODES; do
    run $mode $L $EXTRA
  done
done
if [ "${HYBRID:-0}" = "1" ]; then
  MODEL=llama3-8b
  for mode in odysseus ulysses; do
    run $mode ${HYBRID_L:-262144} --ulysses-degree ${HYBRID_U:-4} --ring-degree ${HYBRID_R:-2} --grad-checkpoint
  done
fi
