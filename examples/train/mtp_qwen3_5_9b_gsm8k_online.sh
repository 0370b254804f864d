#!/bin/bash
# mtp draft for Qwen/Qwen3.5-9B on gsm8k, online hidden states (5k samples: a pipeline check, not a
# production recipe).  Edit the variables or override them in the environment.
set -euo pipefail
export ALGO="${ALGO:-mtp}" MODEL="${MODEL:-Qwen/Qwen3.5-9B}" DATASET="${DATASET:-gsm8k}"
export EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:---num-speculative-steps 3}"
exec bash "$(dirname "$0")/online_pipeline.sh"
