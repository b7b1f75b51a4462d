#!/bin/bash
# The four parallel modes back to back on one 8-GPU box at SEQLEN = GPU_NUM x LOCAL_SEQLEN, as the reference's run.sh does
# (reference run.sh:1-38), on synthetic tokens and random-init Llama-2-7B weights.
LOCAL_SEQLEN=${LOCAL_SEQLEN:-8192}
GPU_NUM=${GPU_NUM:-8}
SEQLEN=$((GPU_NUM*LOCAL_SEQLEN))
MODEL=${MODEL:-llama2-7b}
BACKEND=${BACKEND:-fused}          # fused: own sm_100a kernels + peer-memory collectives; library: torch ops + NCCL
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
# GRADCKP="--grad-checkpoint"

for PARALLEL in ulysses ring odysseus tpsp; do
  python -m torch.distributed.run --nnodes=1 --nproc-per-node=$GPU_NUM --master-addr 127.0.0.1 --master-port 29500 \
    train.py --model-config $MODEL --seq-length $SEQLEN --parallel_mode $PARALLEL --backend $BACKEND $GRADCKP
done
# Ulysses x ring and Odysseus x ring hybrids (inner degree 4, zigzag ring degree 2)
for PARALLEL in ulysses odysseus; do
  python -m torch.distributed.run --nnodes=1 --nproc-per-node=$GPU_NUM --master-addr 127.0.0.1 --master-port 29500 \
    train.py --model-config $MODEL --seq-length $SEQLEN --parallel_mode $PARALLEL --ulysses-degree 4 --ring-degree 2 \
    --backend $BACKEND $GRADCKP
done
