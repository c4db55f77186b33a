#!/bin/bash
# Post-training quantisation of a Llama-2-7B checkpoint on one GPU: calibrate on text (or mock data), print the
# perplexity before and after, save the quantised model (per-rank torch format + quantizer_state.json).
# Recipes: fp8 fp8_blockwise fp8_blockwise_32 int8_sq int4_awq w4a8_awq nvfp4 fp8_real_quant fp8_blockwise_real_quant
# Usage: bash examples/post_training/quantize_llama2_7b.sh <checkpoint dir> <output dir> [recipe] [calibration text file]
set -euo pipefail
CKPT=${1:?checkpoint directory}; OUT=${2:?output directory}; RECIPE=${3:-fp8}; TEXT=${4:-}
[ -n "$TEXT" ] && DATA_ARGS="--valid-data $TEXT --tokenizer-type Llama2Tokenizer --tokenizer-model ${TOKENIZER_MODEL:?set TOKENIZER_MODEL}" \
  || DATA_ARGS="--mock-data --tokenizer-type NullTokenizer --vocab-size 32000"
python -m megatron_lm_b200.tasks.quantize_gpt --load "$CKPT" --save "$OUT" --export-quant-cfg "$RECIPE" \
  --num-layers 32 --hidden-size 4096 --num-attention-heads 32 --ffn-hidden-size 11008 --swiglu \
  --normalization RMSNorm --norm-epsilon 1e-5 --position-embedding-type rope --disable-bias-linear \
  --untie-embeddings-and-output-weights --attention-dropout 0 --hidden-dropout 0 --bf16 \
  --seq-length 4096 --max-position-embeddings 4096 --micro-batch-size 1 \
  --calib-size 128 --calib-batch-size 1 $DATA_ARGS
