#!/bin/bash
# Small GPT (12 layers, hidden 1024, 16 heads, seq 1024, micro-batch 4, global batch 16, fp16, mock data) used to
# exercise rank layouts and the in-memory checkpoint path, with checkpoints in /dev/shm.
#   LAYOUT = tp2pp2 | pp4 | single     (4, 4 or 1 ranks per job)
#   NNODES / NODE_RANK / MASTER_ADDR   for more than one host (defaults: one host, 127.0.0.1)
#   EC=1                               erasure-coded in-memory checkpoint (k data + 1 parity member per stripe)
# Usage: LAYOUT=tp2pp2 bash examples/pre_tests/train_small_gpt.sh [extra flags]
set -euo pipefail
LAYOUT=${LAYOUT:-tp2pp2}
case "$LAYOUT" in
  tp2pp2) PAR="--tensor-model-parallel-size 2 --pipeline-model-parallel-size 2"; WORLD=4 ;;
  pp4)    PAR="--pipeline-model-parallel-size 4"; WORLD=4 ;;
  single) PAR=""; WORLD=1 ;;
  *) echo "unknown LAYOUT $LAYOUT" >&2; exit 2 ;;
esac
NNODES=${NNODES:-1}; NODE_RANK=${NODE_RANK:-0}
PER_NODE=$(( WORLD / NNODES ))
CKPT=${CKPT:-/dev/shm/mlb_pretest_$LAYOUT}
EC_ARGS=""
if [ "${EC:-0}" = "1" ]; then
  EC_ARGS="--non-persistent-ckpt-type local --non-persistent-save-interval 5 --ec-parity-shards 1"
fi
torchrun --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$PER_NODE" \
  --master-addr "${MASTER_ADDR:-127.0.0.1}" --master-port "${MASTER_PORT:-29400}" pretrain_gpt.py $PAR \
  --num-layers 12 --hidden-size 1024 --num-attention-heads 16 --seq-length 1024 --max-position-embeddings 1024 \
  --micro-batch-size 4 --global-batch-size 16 --fp16 --lr 1.5e-4 --min-lr 1e-5 --lr-decay-style cosine \
  --lr-warmup-fraction 0.01 --clip-grad 1.0 --weight-decay 0.01 --train-iters "${TRAIN_ITERS:-50}" \
  --mock-data --tokenizer-type NullTokenizer --vocab-size 50257 --split 949,50,1 \
  --log-interval 5 --eval-interval 1000 --eval-iters 0 --save "$CKPT" --save-interval 25 $EC_ARGS "$@"
