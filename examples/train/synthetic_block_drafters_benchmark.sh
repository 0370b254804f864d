#!/bin/bash
# Step time of DFlash and DSpark training for a Qwen3-8B-shaped verifier, without network or
# server: random-init verifier stub (embeddings, lm_head, norm), synthetic hidden states and
# tokens, the real trainer through the benchmark harness.  Draft: 5 layers, blocks of 16,
# 512 anchors, sliding window 2048 on every layer but the first, hidden states of 5 verifier
# layers, draft vocabulary 32000, packed rows of 4096 tokens.
#
#   bash examples/train/synthetic_block_drafters_benchmark.sh            # 1 GPU
#   NPROC=8 bash examples/train/synthetic_block_drafters_benchmark.sh    # 8 GPUs, sharded optimizer
#
# Every shape is an environment variable, so the same script checks the pipeline on a CPU
# (HIDDEN=128 LAYERS=4 HEADS=2 KV_HEADS=1 HEAD_DIM=64 INTER=256 VOCAB=2048 DRAFT_VOCAB=512 SEQ=512 ...).
set -euo pipefail
WORK="${WORK:-$(mktemp -d)}"
OUT="${OUT:-$WORK}"
ALGOS="${ALGOS:-dflash dspark}"
NPROC="${NPROC:-1}"
HIDDEN="${HIDDEN:-4096}" LAYERS="${LAYERS:-36}" HEADS="${HEADS:-32}" KV_HEADS="${KV_HEADS:-8}" HEAD_DIM="${HEAD_DIM:-128}"
INTER="${INTER:-12288}" VOCAB="${VOCAB:-151936}" DRAFT_VOCAB="${DRAFT_VOCAB:-32000}" SEQ="${SEQ:-4096}"
DRAFT_LAYERS="${DRAFT_LAYERS:-5}" BLOCK="${BLOCK:-16}" ANCHORS="${ANCHORS:-512}" WINDOW="${WINDOW:-2048}"
TARGET_LAYERS="${TARGET_LAYERS:-2 10 18 26 33}"
WARMUP="${WARMUP:-3}" STEPS="${STEPS:-10}"
mkdir -p "$OUT"

python - <<PY
import torch
from speculators_b200.verifier.model import write_random_verifier_stub
cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=$HIDDEN, intermediate_size=$INTER, num_hidden_layers=$LAYERS,
           num_attention_heads=$HEADS, num_key_value_heads=$KV_HEADS, head_dim=$HEAD_DIM, vocab_size=$VOCAB,
           max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1000000.0, hidden_act="silu")
write_random_verifier_stub("$WORK/verifier", cfg, device="cuda" if torch.cuda.is_available() else "cpu")
torch.save({i: $VOCAB - i for i in range($VOCAB)}, "$WORK/token_freq.pt")   # token id -> count: low ids are the frequent ones
PY

if [[ "$NPROC" -gt 1 ]]; then
  LAUNCH=(python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node "$NPROC")
  SHARD=(--fsdp-shard)
else
  LAUNCH=(python)
  SHARD=()
fi

for ALGO in $ALGOS; do
  echo "=== $ALGO ==="
  # shellcheck disable=SC2086
  "${LAUNCH[@]}" scripts/benchmark.py run --synthetic --warmup-steps "$WARMUP" --measured-steps "$STEPS" --no-per-step \
    --output "$OUT/benchmark_$ALGO.json" -- \
    --speculator-type "$ALGO" --verifier-name-or-path "$WORK/verifier" --data-path "$WORK" --save-path "$WORK/ckpt_$ALGO" \
    --token-freq-path "$WORK/token_freq.pt" --draft-vocab-size "$DRAFT_VOCAB" --total-seq-len "$SEQ" \
    --num-layers "$DRAFT_LAYERS" --block-size "$BLOCK" --max-anchors "$ANCHORS" --sliding-window "$WINDOW" --full-attention-indices 0 \
    --target-layer-ids $TARGET_LAYERS --optimizer adamw --lr 1e-4 "${SHARD[@]}"
done
echo "results: $OUT/benchmark_*.json"
