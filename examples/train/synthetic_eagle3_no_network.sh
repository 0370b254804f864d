#!/bin/bash
# Runs anywhere, no model download and no server: a random-init verifier stub and random
# data through the real trainer (the same path the benchmark harness uses).
set -euo pipefail
WORK="${WORK:-$(mktemp -d)}"
python - <<PY
from speculators_b200.verifier.model import write_random_verifier_stub
write_random_verifier_stub("$WORK/verifier", dict(model_type="llama", hidden_size=256, intermediate_size=512, num_hidden_layers=8,
    num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=4096, max_position_embeddings=4096, rms_norm_eps=1e-5))
import torch; torch.save({i: 4096 - i for i in range(4096)}, "$WORK/token_freq.pt")
PY
python scripts/benchmark.py run --synthetic --warmup-steps 3 --measured-steps 10 --output "$WORK/benchmark.json" -- \
  --verifier-name-or-path "$WORK/verifier" --total-seq-len 1024 --draft-vocab-size 1024 --token-freq-path "$WORK/token_freq.pt" \
  --optimizer adamw --lr 1e-4 --save-path "$WORK/ckpt" --data-path "$WORK"
echo "results: $WORK/benchmark.json"
