#!/bin/bash
# EAGLE-3 draft from the original research repository -> this package's checkpoint format,
# loaded once on the GPU afterwards as a check.
set -euo pipefail
python -m speculators_b200 convert yuhuili/EAGLE3-LLaMA3.1-Instruct-8B --algorithm eagle3 \
    --verifier meta-llama/Meta-Llama-3.1-8B-Instruct --output-path ./eagle3-llama-3.1-8b-instruct-converted \
    --validate-device cuda:0
