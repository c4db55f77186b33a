#!/bin/bash
# Distil a smaller student from a frozen Llama-2-7B teacher on 8 GPUs (TP4 x DP2).  The teacher's architecture is read
# from <teacher checkpoint>/model_config.yaml (num_layers, hidden_size, ffn_hidden_size, num_attention_heads, ...);
# without that file the teacher has the student's architecture.
# Usage: bash examples/post_training/distill_llama.sh <teacher checkpoint> <data-prefix|--mock-data> [extra flags]
set -euo pipefail
TEACHER=${1:?teacher checkpoint}; DATA=${2:---mock-data}; shift 2 || true
[ "$DATA" = "--mock-data" ] && DATA_ARGS="--mock-data --tokenizer-type NullTokenizer --vocab-size 32000" \
  || DATA_ARGS="--data-path $DATA --tokenizer-type Llama2Tokenizer --tokenizer-model ${TOKENIZER_MODEL:?set TOKENIZER_MODEL}"
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_gpt.py \
  --export-kd-teacher-load "$TEACHER" --export-kd-cfg examples/post_training/distill.yaml \
  --tensor-model-parallel-size 4 --sequence-parallel --use-distributed-optimizer --overlap-grad-reduce \
  --num-layers 16 --hidden-size 2048 --num-attention-heads 16 --ffn-hidden-size 5504 --swiglu \
  --normalization RMSNorm --position-embedding-type rope --disable-bias-linear --untie-embeddings-and-output-weights \
  --attention-dropout 0 --hidden-dropout 0 --seq-length 4096 --max-position-embeddings 4096 \
  --micro-batch-size 1 --global-batch-size 64 --bf16 --lr 1e-4 --min-lr 1e-5 --lr-decay-style cosine \
  --train-iters 1000 --log-interval 10 --eval-interval 1000 --eval-iters 0 $DATA_ARGS "$@"
