#!/bin/bash
# GPT-3 1.3B: TP2 x DP4 with sequence parallelism and the distributed optimizer on 8 GPUs.
set -euo pipefail
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_gpt.py \
  --tensor-model-parallel-size 2 --sequence-parallel --use-distributed-optimizer --overlap-grad-reduce \
  --overlap-param-gather --tp-comm-overlap --num-layers 24 --hidden-size 2048 --num-attention-heads 16 \
  --seq-length 2048 --max-position-embeddings 2048 --micro-batch-size 4 --global-batch-size 256 --bf16 \
  --lr 2e-4 --min-lr 2e-5 --lr-decay-style cosine --weight-decay 0.1 --clip-grad 1.0 --init-method-std 0.02 \
  --train-iters 1000 --log-interval 10 --eval-iters 0 --split 100,0,0 \
  --mock-data --tokenizer-type NullTokenizer --vocab-size 50304 "$@"
