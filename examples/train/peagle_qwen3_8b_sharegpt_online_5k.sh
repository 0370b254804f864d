#!/bin/bash
# peagle draft for Qwen/Qwen3-8B on sharegpt, online hidden states (5k samples: a pipeline check, not a
# production recipe).  Edit the variables or override them in the environment.
set -euo pipefail
export ALGO="${ALGO:-peagle}" MODEL="${MODEL:-Qwen/Qwen3-8B}" DATASET="${DATASET:-sharegpt}"
export EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:---num-depths 8 --max-anchors 2048}"
exec bash "$(dirname "$0")/online_pipeline.sh"
