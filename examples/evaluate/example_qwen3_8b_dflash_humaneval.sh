#!/bin/bash
# Acceptance rates of a DFlash draft on HumaneEval prompts: serve the verifier with the draft
# attached, run the throughput-mode evaluation, print the acceptance report.
set -euo pipefail
MODEL="${MODEL:-Qwen/Qwen3-8B}"
DRAFT="${DRAFT:-./checkpoints/dflash/checkpoint_best}"
PORT="${PORT:-8000}"
python -m vllm.entrypoints.cli.main serve "$MODEL" --port "$PORT" \
  --speculative-config "{\"model\": \"$DRAFT\", \"num_speculative_tokens\": 7}" &
server=$!
trap 'kill "$server" 2>/dev/null || true; wait "$server" 2>/dev/null || true' EXIT
until curl -sf "http://localhost:${PORT}/health" > /dev/null 2>&1; do sleep 2; done
python scripts/evaluate/evaluate.py --target "http://localhost:${PORT}/v1" throughput --subsets HumanEval --output-dir ./eval_dflash_humaneval
cat ./eval_dflash_humaneval/acceptance.csv
