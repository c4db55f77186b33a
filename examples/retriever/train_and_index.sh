#!/bin/bash
# Retriever: inverse-cloze-task training of a biencoder, then the evidence file embedded by its context tower.
# Usage: bash examples/retriever/train_and_index.sh <sentence-split corpus prefix> <title prefix> <vocab.txt> <evidence.tsv> <work dir>
# The evidence file has a header line and then `id <tab> text <tab> title` per row.
set -euo pipefail
DATA=${1:?corpus prefix}; TITLES=${2:?title prefix}; VOCAB=${3:?vocab file}; EVIDENCE=${4:?evidence tsv}; WORK=${5:?work dir}
MODEL="--num-layers 12 --hidden-size 768 --num-attention-heads 12 --seq-length 256 --max-position-embeddings 512 \
  --retriever-seq-length 256 --biencoder-projection-dim 128 --tokenizer-type BertWordPieceLowerCase --vocab-file $VOCAB --bf16"
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 pretrain_ict.py $MODEL \
  --data-path "$DATA" --titles-data-path "$TITLES" --split 949,50,1 --query-in-block-prob 0.1 \
  --retriever-report-topk-accuracies 1 5 20 --retriever-score-scaling \
  --micro-batch-size 32 --global-batch-size 256 --lr 1e-4 --min-lr 1e-6 --lr-decay-style linear --lr-warmup-fraction 0.01 \
  --weight-decay 0.01 --clip-grad 1.0 --train-iters 100000 --log-interval 100 --eval-interval 1000 --eval-iters 10 \
  --save "$WORK/ict" --save-interval 5000
torchrun --nnodes 1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 -m megatron_lm_b200.tasks.build_evidence_index $MODEL \
  --micro-batch-size 32 --ict-load "$WORK/ict" --evidence-data-path "$EVIDENCE" --embedding-path "$WORK/evidence_embeds.pt" \
  --indexer-batch-size 128 --indexer-log-interval 1000
