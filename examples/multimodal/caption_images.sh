#!/bin/bash
# Generate text for every image of a folder with a LLaVA-style model (CLIP ViT-L/14 at 336 px + Llama-2-7B shown here).
# A Hugging Face LLaVA checkpoint is converted first with:
#   python -m megatron_lm_b200.checkpoint.convert --loader llava_hf --saver core --load-dir <hf dir> --save-dir <ckpt>
# Usage: bash examples/multimodal/caption_images.sh <checkpoint dir> <image folder> <output.jsonl> [extra flags]
set -euo pipefail
CKPT=${1:?checkpoint directory}; IMAGES=${2:?image folder}; OUT=${3:?output file}; shift 3 || true
python -m megatron_lm_b200.inference.run_vlm_generation --load "$CKPT" --input-image-path "$IMAGES" --output-path "$OUT" \
  --prompt "<image>\nDescribe the image in one sentence." --out-seq-length 48 --top-k 1 \
  --num-layers 32 --hidden-size 4096 --num-attention-heads 32 --ffn-hidden-size 11008 --swiglu \
  --normalization RMSNorm --position-embedding-type rope --disable-bias-linear --untie-embeddings-and-output-weights \
  --encoder-num-layers 23 --img-h 336 --img-w 336 --patch-dim 14 --disable-vision-class-token \
  --seq-length 2048 --max-position-embeddings 4096 --bf16 --tokenizer-type Llama2Tokenizer \
  --tokenizer-model "${TOKENIZER_MODEL:?set TOKENIZER_MODEL}" "$@"
