#!/bin/bash
# Second half of the recovery exercise: run train_small_gpt.sh first (it leaves checkpoints in /dev/shm), then this
# script resumes from them and trains further.  Same LAYOUT / NNODES / EC variables.
set -euo pipefail
LAYOUT=${LAYOUT:-tp2pp2}
CKPT=${CKPT:-/dev/shm/mlb_pretest_$LAYOUT}
[ -f "$CKPT/latest_checkpointed_iteration.txt" ] || { echo "no checkpoint under $CKPT" >&2; exit 1; }
TRAIN_ITERS=${TRAIN_ITERS:-100} CKPT=$CKPT LAYOUT=$LAYOUT \
  bash "$(dirname "$0")/train_small_gpt.sh" --load "$CKPT" "$@"
