#!/bin/bash
# Mixtral-style 8-expert top-2 MoE, expert parallel over 8 GPUs (reference counterpart:
# examples/mixtral/train_mixtral_8x7b_distributed.sh).  16 layers fit one node; raise --num-layers with more nodes.
set -euo pipefail
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_gpt.py \
  --expert-model-parallel-size 8 --use-distributed-optimizer --overlap-grad-reduce \
  --num-layers 16 --hidden-size 4096 --num-attention-heads 32 --group-query-attention --num-query-groups 8 \
  --ffn-hidden-size 14336 --swiglu --normalization RMSNorm --position-embedding-type rope --rotary-base 1000000 \
  --disable-bias-linear --untie-embeddings-and-output-weights --attention-dropout 0 --hidden-dropout 0 \
  --num-experts 8 --moe-router-topk 2 --moe-router-load-balancing-type aux_loss --moe-aux-loss-coeff 1e-2 \
  --moe-token-dispatcher-type alltoall --moe-grouped-gemm \
  --seq-length 4096 --max-position-embeddings 4096 --micro-batch-size 1 --global-batch-size 64 --bf16 \
  --lr 1e-4 --min-lr 1e-5 --lr-decay-style cosine --weight-decay 0.1 --clip-grad 1.0 --init-method-std 0.02 \
  --train-iters 1000 --log-interval 10 --eval-iters 0 --split 100,0,0 \
  --mock-data --tokenizer-type NullTokenizer --vocab-size 32000 "$@"
