#!/usr/bin/env bash
# Generation smoke test.  MODEL_PATH=/path/to/hub [LORA_PATH=output_sft/...] ./run_test_generation.sh
set -euo pipefail
cd "$(dirname "$0")"
: "${MODEL_PATH:?set MODEL_PATH to a model hub directory}"
ARGS=(--model_path "$MODEL_PATH"
      --data_file "${DATA_FILE:-data/sharegpt_sample.jsonl}"
      --num_samples "${NUM_SAMPLES:-3}"
      --max_new_tokens "${MAX_NEW_TOKENS:-256}"
      --temperature "${TEMPERATURE:-0.8}"
      --top_p "${TOP_P:-0.9}"
      --repetition_penalty "${REPETITION_PENALTY:-1.0}"
      --device "${DEVICE:-cuda}")
[[ -n "${LORA_PATH:-}" ]] && ARGS+=(--lora_path "$LORA_PATH")
[[ -n "${OUTPUT_JSON:-}" ]] && ARGS+=(--output_json "$OUTPUT_JSON")
CUDA_VISIBLE_DEVICES="${GPU_ID:-0}" exec python test_generation.py "${ARGS[@]}"
