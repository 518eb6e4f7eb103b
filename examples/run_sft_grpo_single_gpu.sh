#!/usr/bin/env bash
# SFT (LoRA), merge the adapter into a new hub, then GRPO on the merged model.
set -euo pipefail
cd "$(dirname "$0")"
: "${MODEL_PATH:?set MODEL_PATH to a model hub directory}"
WORK="${WORK_DIR:-output_sft_grpo}"
USE_LORA=1 OUTPUT_DIR="$WORK/sft" ./run_sft_single_gpu.sh
ADAPTER="$(ls -d "$WORK"/sft/*/ 2>/dev/null | sort | tail -n 1)"
python -m rwkvtune_b200.cli.merge_lora --base-model "$MODEL_PATH" --lora-model "${ADAPTER:-$WORK/sft}" --output "$WORK/merged"
MODEL_PATH="$WORK/merged" OUTPUT_DIR="$WORK/grpo" ./run_grpo_single_gpu.sh
