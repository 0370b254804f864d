#!/bin/bash
# eagle3 draft for Qwen/Qwen3-8B on sharegpt, online hidden states (5k samples: a pipeline check, not a
# production recipe).  Edit the variables or override them in the environment.
set -euo pipefail
export ALGO="${ALGO:-eagle3}" MODEL="${MODEL:-Qwen/Qwen3-8B}" DATASET="${DATASET:-sharegpt}"
export EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:---ttt-steps 3}"
exec bash "$(dirname "$0")/online_pipeline.sh"
