#!/bin/bash
# Llama-2-7B pre-training on one 8 x B200 node: TP4 x PP2 (2 virtual stages), sequence parallel,
# distributed optimizer, fused TP kernels, bf16.  Pass --fp8-format hybrid --fp8-recipe tensorwise for FP8 GEMMs.
# Usage: bash examples/llama/train_llama2_7b_b200.sh <data-prefix|--mock-data> [extra flags]
set -euo pipefail
DATA=${1:---mock-data}; shift || true
[ "$DATA" = "--mock-data" ] && DATA_ARGS="--mock-data --tokenizer-type NullTokenizer --vocab-size 32000" \
  || DATA_ARGS="--data-path $DATA --tokenizer-type Llama2Tokenizer --tokenizer-model ${TOKENIZER_MODEL:?set TOKENIZER_MODEL}"
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_gpt.py \
  --tensor-model-parallel-size 4 --pipeline-model-parallel-size 2 --num-layers-per-virtual-pipeline-stage 8 \
  --sequence-parallel --use-distributed-optimizer --overlap-grad-reduce --overlap-param-gather --tp-comm-overlap \
  --num-layers 32 --hidden-size 4096 --num-attention-heads 32 --ffn-hidden-size 11008 --swiglu \
  --normalization RMSNorm --norm-epsilon 1e-5 --position-embedding-type rope --rotary-base 10000 \
  --disable-bias-linear --untie-embeddings-and-output-weights --attention-dropout 0 --hidden-dropout 0 \
  --seq-length 4096 --max-position-embeddings 4096 --micro-batch-size 1 --global-batch-size 64 \
  --bf16 --lr 3e-4 --min-lr 3e-5 --lr-decay-style cosine --lr-warmup-iters 200 --weight-decay 0.1 --clip-grad 1.0 \
  --adam-beta1 0.9 --adam-beta2 0.95 --init-method-std 0.02 --train-iters 1000 --log-interval 10 \
  --eval-interval 1000 --eval-iters 0 --split 100,0,0 $DATA_ARGS "$@"
