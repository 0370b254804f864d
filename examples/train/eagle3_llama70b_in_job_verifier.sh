#!/bin/bash
# EAGLE-3 draft for a 70B-class dense verifier with the verifier inside the training job: no
# server, no hidden-state files.  The first VERIFIER_GPUS ranks load the checkpoint tensor-parallel
# and run the packed rows of the dataset; the other ranks train on the hidden states that arrive
# in their NVLink rings (docs/user_guide/tutorials/train.md, "Online training with the verifier
# inside the job").
#
#   MODEL=/models/Llama-3.3-70B-Instruct DATA=./output bash examples/train/eagle3_llama70b_in_job_verifier.sh
#
# DATA is the output of scripts/prepare_data.py (input_ids / loss_mask / seq_len) plus the vocabulary
# mapping of scripts/build_vocab_mapping.py; MODEL must be a local directory with config.json and
# safetensors shards.  The tensor-parallel size has to divide the verifier's attention and KV head counts.
set -euo pipefail

MODEL="${MODEL:?path of the verifier checkpoint}"
DATA="${DATA:-./output}"
SAVE_DIR="${SAVE_DIR:-./checkpoints/eagle3_in_job}"
GPUS="${GPUS:-8}"
VERIFIER_GPUS="${VERIFIER_GPUS:-4}"
SEQ_LENGTH="${SEQ_LENGTH:-8192}"
EPOCHS="${EPOCHS:-5}"
LR="${LR:-1e-4}"
DRAFT_VOCAB_SIZE="${DRAFT_VOCAB_SIZE:-32000}"
EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:-}"

# shellcheck disable=SC2086
torchrun --standalone --nproc_per_node "$GPUS" scripts/train.py \
    --speculator-type eagle3 --verifier-name-or-path "$MODEL" --data-path "$DATA" \
    --online-verifier-gpus "$VERIFIER_GPUS" --online-ring-slots 4 \
    --draft-vocab-size "$DRAFT_VOCAB_SIZE" --total-seq-len "$SEQ_LENGTH" --epochs "$EPOCHS" --lr "$LR" \
    --optimizer adamw --fsdp-shard --save-path "$SAVE_DIR" $EXTRA_TRAIN_ARGS
