#!/bin/bash
# Start an 8-expert mixture-of-experts run from a dense checkpoint (--moe-use-upcycling): every expert begins as a copy
# of the dense MLP (a 1/g slice with --moe-upcycling-granularity g), routers start from small random values.
# Usage: bash examples/post_training/upcycle_to_moe.sh <dense checkpoint> <new checkpoint dir> [extra flags]
set -euo pipefail
DENSE=${1:?dense checkpoint}; OUT=${2:?output directory}; shift 2 || true
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_gpt.py \
  --moe-use-upcycling --load "$DENSE" --save "$OUT" --save-interval 500 \
  --expert-model-parallel-size 8 --num-experts 8 --moe-router-topk 2 --moe-grouped-gemm --moe-aux-loss-coeff 1e-2 \
  --moe-token-dispatcher-type alltoall --use-distributed-optimizer \
  --num-layers 32 --hidden-size 4096 --num-attention-heads 32 --ffn-hidden-size 11008 --swiglu \
  --normalization RMSNorm --position-embedding-type rope --disable-bias-linear --untie-embeddings-and-output-weights \
  --attention-dropout 0 --hidden-dropout 0 --seq-length 4096 --max-position-embeddings 4096 \
  --micro-batch-size 1 --global-batch-size 64 --bf16 --lr 1e-4 --min-lr 1e-5 --lr-decay-style cosine \
  --train-iters 1000 --log-interval 10 --eval-interval 1000 --eval-iters 0 \
  --mock-data --tokenizer-type NullTokenizer --vocab-size 32000 "$@"
