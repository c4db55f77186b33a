#!/bin/bash
# Four "nodes" of one GPU each on a single host: one torchrun per node, each pinned to its own GPU, all joining
# one rendezvous.  Exercises the multi-node code paths (node ranks, cross-"node" groups) without a cluster.
# Usage: bash examples/pre_tests/fake_nodes.sh [pretrain_gpt.py flags]
set -euo pipefail
NODES=${NODES:-4}
PORT=${MASTER_PORT:-29410}
pids=()
for n in $(seq 0 $(( NODES - 1 ))); do
  CUDA_VISIBLE_DEVICES=$n torchrun --nnodes "$NODES" --node-rank "$n" --nproc-per-node 1 \
    --master-addr 127.0.0.1 --master-port "$PORT" pretrain_gpt.py --pipeline-model-parallel-size "$NODES" \
    --num-layers 12 --hidden-size 1024 --num-attention-heads 16 --seq-length 1024 --max-position-embeddings 1024 \
    --micro-batch-size 4 --global-batch-size 16 --fp16 --lr 1.5e-4 --train-iters "${TRAIN_ITERS:-20}" \
    --mock-data --tokenizer-type NullTokenizer --vocab-size 50257 --log-interval 5 --eval-iters 0 "$@" \
    > "fake_node_$n.log" 2>&1 &
  pids+=($!)
done
rc=0
for p in "${pids[@]}"; do wait "$p" || rc=$?; done
exit $rc
