#!/bin/bash
# Vision transformer pre-training on 8 GPUs (data parallel): supervised classification, DINO self-distillation or
# in-painting.  Data: <root>/train/<class>/*.npy|png|jpg and <root>/val/..., or --mock-data.
# Usage: bash examples/vision/pretrain_vit.sh <classify|dino|inpaint> <image root|--mock-data> [extra flags]
# Other backbones: append `--vision-backbone-type mit` (classify, dino; inpaint with `--patch-dim 4`) or
# `--vision-backbone-type swin --swin-backbone-type tiny|base|h3` (dino).
set -euo pipefail
TASK=${1:?classify, dino or inpaint}; DATA=${2:---mock-data}; shift 2 || true
[ "$DATA" = "--mock-data" ] && DATA_ARGS="--mock-data" || DATA_ARGS="--data-path $DATA"
case "$TASK" in
  classify) EXTRA="--num-classes 1000 --head-lr-mult 1.0" ;;
  dino)     EXTRA="--dino-local-crops-number 8 --dino-local-img-size 96 --dino-head-hidden-size 2048 --dino-bottleneck-size 256 --dino-out-dim 65536 --iter-per-epoch 1250 --dino-warmup-teacher-temp-epochs 30 --dino-freeze-last-layer 1 --num-classes 1000" ;;
  inpaint)  EXTRA="--mask-type random --mask-factor 1.0 --num-classes 1000" ;;
  *) echo "unknown task $TASK"; exit 1 ;;
esac
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_vision_$TASK.py \
  --num-layers 12 --hidden-size 768 --num-attention-heads 12 --seq-length 197 --max-position-embeddings 197 \
  --img-h 224 --img-w 224 --patch-dim 16 --attention-dropout 0 --hidden-dropout 0 \
  --micro-batch-size 64 --global-batch-size 512 --bf16 --lr 5e-4 --min-lr 1e-6 --lr-decay-style cosine \
  --lr-warmup-fraction 0.05 --weight-decay 0.05 --clip-grad 1.0 --use-distributed-optimizer --overlap-grad-reduce \
  --train-iters 10000 --log-interval 20 --eval-interval 1000 --eval-iters 10 $EXTRA $DATA_ARGS "$@"
