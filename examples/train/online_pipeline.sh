#!/bin/bash
# Online training pipeline: prepare data, start the verifier server with hidden-state
# extraction, train a draft model while hidden states are generated on the fly.
#
#   ALGO=eagle3 MODEL=Qwen/Qwen3-8B DATASET=sharegpt bash examples/train/online_pipeline.sh
#
# Every setting is an environment variable with a default; the per-algorithm scripts in
# this folder only set them.  The data must hold responses of the target model itself
# (see scripts/response_regeneration/ for how to regenerate them).
set -euo pipefail

ALGO="${ALGO:-eagle3}"                    # eagle3 | peagle | dflash | dspark | mtp
MODEL="${MODEL:-Qwen/Qwen3-8B}"
DATASET="${DATASET:-sharegpt}"            # preset name, .jsonl file, directory or hf:<id>
OUTPUT_DIR="${OUTPUT_DIR:-./output}"
SAVE_DIR="${SAVE_DIR:-./checkpoints/$ALGO}"
VLLM_PORT="${VLLM_PORT:-8000}"
VLLM_GPUS="${VLLM_GPUS:-0,1}"             # the server and the trainer need separate GPUs
TRAIN_GPUS="${TRAIN_GPUS:-2,3}"
NUM_TRAIN_GPUS="${NUM_TRAIN_GPUS:-2}"
VLLM_ARGS="${VLLM_ARGS:---data-parallel-size 2 --gpu-memory-utilization 0.85}"
LAUNCH_ARGS="${LAUNCH_ARGS:-}"            # flags of scripts/launch_vllm.py itself, e.g. --target-layer-ids 2 18 33
DRAFT_VOCAB_SIZE="${DRAFT_VOCAB_SIZE:-32000}"
MAX_SAMPLES="${MAX_SAMPLES:-5000}"
SEQ_LENGTH="${SEQ_LENGTH:-8192}"
EPOCHS="${EPOCHS:-5}"
LR="${LR:-1e-4}"
EXTRA_TRAIN_ARGS="${EXTRA_TRAIN_ARGS:-}"  # algorithm-specific flags

echo "=== 1/4 starting the verifier server ($MODEL on GPUs $VLLM_GPUS) ==="
# shellcheck disable=SC2086
CUDA_VISIBLE_DEVICES="$VLLM_GPUS" python scripts/launch_vllm.py "$MODEL" $LAUNCH_ARGS -- --port "$VLLM_PORT" $VLLM_ARGS &
server=$!
trap 'kill "$server" 2>/dev/null || true; wait "$server" 2>/dev/null || true' EXIT
until curl -sf "http://localhost:${VLLM_PORT}/health" > /dev/null 2>&1; do
  kill -0 "$server" 2>/dev/null || { echo "the server exited early" >&2; exit 1; }
  sleep 2
done

echo "=== 2/4 preparing data (render-boundary loss masks through the server) ==="
python scripts/prepare_data.py --model "$MODEL" --data "$DATASET" --output "$OUTPUT_DIR" \
  --max-samples "$MAX_SAMPLES" --seq-length "$SEQ_LENGTH" --render-endpoint "http://localhost:${VLLM_PORT}"

if [[ "$ALGO" != "mtp" ]]; then
  echo "=== 3/4 building the draft vocabulary ==="
  python scripts/build_vocab_mapping.py --token-freq-path "$OUTPUT_DIR/token_freq.pt" \
    --draft-vocab-size "$DRAFT_VOCAB_SIZE" --target-model-path "$MODEL" --output-path "$OUTPUT_DIR"
fi

echo "=== 4/4 training ($ALGO, $NUM_TRAIN_GPUS GPUs) ==="
# shellcheck disable=SC2086
CUDA_VISIBLE_DEVICES="$TRAIN_GPUS" torchrun --standalone --local-addr 127.0.0.1 --nproc_per_node "$NUM_TRAIN_GPUS" scripts/train.py \
  --speculator-type "$ALGO" --verifier-name-or-path "$MODEL" --data-path "$OUTPUT_DIR" --save-path "$SAVE_DIR" \
  --vllm-endpoint "http://localhost:${VLLM_PORT}/v1" --on-missing generate --on-generate delete \
  --total-seq-len "$SEQ_LENGTH" --epochs "$EPOCHS" --lr "$LR" --optimizer adamw --fsdp-shard \
  $( [[ "$ALGO" != "mtp" ]] && echo --draft-vocab-size "$DRAFT_VOCAB_SIZE" ) $EXTRA_TRAIN_ARGS
echo "checkpoints in $SAVE_DIR (load with vLLM: --speculative-config '{\"model\": \"$SAVE_DIR/checkpoint_best\"}')"
