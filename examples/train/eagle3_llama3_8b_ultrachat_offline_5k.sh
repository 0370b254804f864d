#!/bin/bash
# Offline variant: hidden states are generated once into files, the server is stopped, then
# training reads them from disk (all GPUs free for training).
set -euo pipefail
MODEL="${MODEL:-meta-llama/Llama-3.1-8B-Instruct}"
DATASET="${DATASET:-ultrachat}"
OUTPUT_DIR="${OUTPUT_DIR:-./output}"
SAVE_DIR="${SAVE_DIR:-./checkpoints/eagle3}"
VLLM_PORT="${VLLM_PORT:-8000}"
NUM_GPUS="${NUM_GPUS:-4}"

python scripts/launch_vllm.py "$MODEL" --hidden-states-path "$OUTPUT_DIR/tmp_hidden_states" -- --port "$VLLM_PORT" --data-parallel-size "$NUM_GPUS" &
server=$!
trap 'kill "$server" 2>/dev/null || true; wait "$server" 2>/dev/null || true' EXIT
until curl -sf "http://localhost:${VLLM_PORT}/health" > /dev/null 2>&1; do sleep 2; done
python scripts/prepare_data.py --model "$MODEL" --data "$DATASET" --output "$OUTPUT_DIR" --max-samples 5000 \
  --render-endpoint "http://localhost:${VLLM_PORT}"
python scripts/data_generation_offline.py --preprocessed-data "$OUTPUT_DIR" --endpoint "http://localhost:${VLLM_PORT}/v1" \
  --concurrency 32 --validate-outputs
kill "$server"; wait "$server" 2>/dev/null || true; trap - EXIT
python scripts/build_vocab_mapping.py --token-freq-path "$OUTPUT_DIR/token_freq.pt" --draft-vocab-size 32000 \
  --target-model-path "$MODEL" --output-path "$OUTPUT_DIR"
torchrun --standalone --local-addr 127.0.0.1 --nproc_per_node "$NUM_GPUS" scripts/train.py --speculator-type eagle3 \
  --verifier-name-or-path "$MODEL" --data-path "$OUTPUT_DIR" --save-path "$SAVE_DIR" --on-missing raise \
  --epochs 5 --lr 1e-4 --optimizer adamw --fsdp-shard --draft-vocab-size 32000
