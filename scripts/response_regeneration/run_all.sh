#!/bin/bash
# Start a vLLM server for the target model, regenerate a dataset's responses with it,
# stop the server again.
#
#   ./run_all.sh --model meta-llama/Llama-3.3-70B-Instruct --dataset magpie --limit 100
#   ./run_all.sh --model Qwen/Qwen2.5-72B-Instruct --dp-size 4 --tp-size 2 --dataset magpie
#   ./run_all.sh --model Qwen/Qwen3-8B --tool-call-parser hermes --dataset hermes-fc --keep-server
#
# Server flags: --model --port --dp-size --tp-size --max-model-len --reasoning-parser
# --tool-call-parser --gpus (CUDA_VISIBLE_DEVICES list) --keep-server.  Every other
# argument goes to script.py.
set -euo pipefail

here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
port=8000 model="" dp="" tp="" max_len="" reasoning="" tool_parser="" gpus="" keep=false
passthrough=()
while [[ $# -gt 0 ]]; do
  case "$1" in
    --port) port="$2"; shift 2 ;;
    --model) model="$2"; shift 2 ;;
    --dp-size) dp="$2"; shift 2 ;;
    --tp-size) tp="$2"; shift 2 ;;
    --max-model-len) max_len="$2"; shift 2 ;;
    --reasoning-parser) reasoning="$2"; shift 2 ;;
    --tool-call-parser) tool_parser="$2"; shift 2 ;;
    --gpus) gpus="$2"; shift 2 ;;
    --keep-server) keep=true; shift ;;
    *) passthrough+=("$1"); shift ;;
  esac
done
[[ -n "$model" ]] || { echo "--model is required" >&2; exit 2; }

serve=(python -m vllm.entrypoints.cli.main serve "$model" --port "$port")
[[ -n "$dp" ]] && serve+=(--data-parallel-size "$dp")
[[ -n "$tp" ]] && serve+=(--tensor-parallel-size "$tp")
[[ -n "$max_len" ]] && serve+=(--max-model-len "$max_len")
[[ -n "$reasoning" ]] && serve+=(--reasoning-parser "$reasoning")
[[ -n "$tool_parser" ]] && serve+=(--enable-auto-tool-choice --tool-call-parser "$tool_parser")

log="vllm_server_${port}.log"
echo "Starting server: ${serve[*]} (log: $log)"
if [[ -n "$gpus" ]]; then CUDA_VISIBLE_DEVICES="$gpus" "${serve[@]}" > "$log" 2>&1 & else "${serve[@]}" > "$log" 2>&1 & fi
server_pid=$!
stop_server() { if [[ "$keep" == false ]]; then echo "Stopping server ($server_pid)"; kill "$server_pid" 2>/dev/null || true; wait "$server_pid" 2>/dev/null || true; fi; }
trap stop_server EXIT

echo "Waiting for the server on port $port ..."
for _ in $(seq 1 360); do
  if curl -sf "http://127.0.0.1:${port}/v1/models" > /dev/null; then break; fi
  if ! kill -0 "$server_pid" 2>/dev/null; then echo "Server exited early; see $log" >&2; exit 1; fi
  sleep 5
done
curl -sf "http://127.0.0.1:${port}/v1/models" > /dev/null || { echo "Server did not come up; see $log" >&2; exit 1; }

python "$here/script.py" --endpoint "http://127.0.0.1:${port}/v1/chat/completions" --model "$model" "${passthrough[@]}"
