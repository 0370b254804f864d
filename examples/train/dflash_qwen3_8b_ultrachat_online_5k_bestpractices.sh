#!/bin/bash
# dflash draft for Qwen/Qwen3-8B on ultrachat with the recommended recipe: five draft layers,
# blocks of 16 positions, cross-entropy loss with D-PACE per-position weights, verifier
# layers 2 / 18 / 33 as draft input.  These are also what `--speculator-type dflash` picks by
# default; they are spelled out so the script documents the whole recipe.  5k samples check
# the pipeline, they do not make a good draft.  Edit the variables or override them in the
# environment.
set -euo pipefail
TARGET_LAYER_IDS="${TARGET_LAYER_IDS:-2 18 33}"   # must equal the server's auxiliary hidden-state layers
export ALGO="${ALGO:-dflash}" MODEL="${MODEL:-Qwen/Qwen3-8B}" DATASET="${DATASET:-ultrachat}"
export OUTPUT_DIR="${OUTPUT_DIR:-./output/dflash_qwen3_8b_ultrachat_bestpractices}" LR="${LR:-3e-4}"
export LAUNCH_ARGS="${LAUNCH_ARGS:---target-layer-ids $TARGET_LAYER_IDS}"
export EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:---num-layers 5 --block-size 16 --max-anchors 3072 --loss-fn ce --per-position-loss-weight dpace --target-layer-ids $TARGET_LAYER_IDS}"
exec bash "$(dirname "$0")/online_pipeline.sh"
