#!/bin/bash
# dspark draft for Qwen/Qwen3-0.6B on sharegpt, online hidden states (5k samples: a pipeline check, not a
# production recipe).  Edit the variables or override them in the environment.
set -euo pipefail
export ALGO="${ALGO:-dspark}" MODEL="${MODEL:-Qwen/Qwen3-0.6B}" DATASET="${DATASET:-sharegpt}"
export EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:---block-size 8 --max-anchors 512 --markov-rank 256}"
exec bash "$(dirname "$0")/online_pipeline.sh"
