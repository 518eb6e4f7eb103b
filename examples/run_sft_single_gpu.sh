#!/usr/bin/env bash
# SFT on one GPU.  Every setting is an environment variable with a default:
#   MODEL_PATH=/path/to/hub CTX_LEN=1024 MICRO_BSZ=4 USE_LORA=1 ./run_sft_single_gpu.sh
set -euo pipefail
cd "$(dirname "$0")"
: "${MODEL_PATH:?set MODEL_PATH to a model hub directory}"
ARGS=(--model_path "$MODEL_PATH"
      --data_file "${DATA_FILE:-data/sharegpt_sample.jsonl}"
      --output_dir "${OUTPUT_DIR:-output_sft}"
      --ctx_len "${CTX_LEN:-2048}"
      --micro_bsz "${MICRO_BSZ:-2}"
      --accumulate_grad_batches "${ACCUMULATE_GRAD_BATCHES:-4}"
      --epoch_count "${EPOCHS:-3}"
      --lr_init "${LR_INIT:-2e-5}"
      --lr_final "${LR_FINAL:-1e-6}"
      --warmup_steps "${WARMUP_STEPS:-10}"
      --precision "${PRECISION:-bf16}"
      --epoch_save "${EPOCH_SAVE:-1}"
      --save_total_limit "${SAVE_TOTAL_LIMIT:-3}")
if [[ "${USE_LORA:-0}" == "1" ]]; then
  ARGS+=(--use_lora --lora_r "${LORA_R:-64}" --lora_alpha "${LORA_ALPHA:-128}" --lora_dropout "${LORA_DROPOUT:-0.0}")
fi
[[ "${LAST_REPLY_ONLY:-0}" == "1" ]] && ARGS+=(--last_reply_only)
[[ -n "${ACCELERATOR:-}" ]] && ARGS+=(--accelerator "$ACCELERATOR")      # ACCELERATOR=cpu PRECISION=fp32 runs on the host
[[ -n "${REPORT_TO:-}" ]] && ARGS+=(--report_to "$REPORT_TO" --run_name "${RUN_NAME:-sft}")
CUDA_VISIBLE_DEVICES="${GPU_ID:-0}" exec python train_sft_single_gpu.py "${ARGS[@]}"
