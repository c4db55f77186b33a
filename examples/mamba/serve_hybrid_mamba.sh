#!/bin/bash
# Serve a hybrid Mamba-2 / attention model over HTTP (PUT /api, the request format of the GPT server) with the static
# engine; query it with: python -m megatron_lm_b200.inference.cli 127.0.0.1:5000 --prompt "..." --tokens-to-generate 64
# Usage: bash examples/mamba/serve_hybrid_mamba.sh <checkpoint dir> [extra flags]
set -euo pipefail
CKPT=${1:?checkpoint directory}; shift || true
python -m megatron_lm_b200.inference.run_server --server-model-type mamba --load "$CKPT" \
  --num-layers 56 --hidden-size 4096 --num-attention-heads 32 --group-query-attention --num-query-groups 8 \
  --hybrid-override-pattern "M-M-M-M*-M-M-M-M-M*-M-M-M-M-M*-M-M-M-M-M*-M-M-M-M-M-" \
  --mamba-state-dim 128 --mamba-head-dim 64 --mamba-num-groups 8 --ffn-hidden-size 14336 --squared-relu \
  --normalization RMSNorm --position-embedding-type none --disable-bias-linear --untie-embeddings-and-output-weights \
  --seq-length 4096 --max-position-embeddings 4096 --bf16 --tokenizer-type HuggingFaceTokenizer \
  --tokenizer-model "${TOKENIZER_MODEL:?set TOKENIZER_MODEL}" --inference-max-requests 8 --port 5000 "$@"
