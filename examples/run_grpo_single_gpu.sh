#!/usr/bin/env bash
# GRPO (LoRA) on one GPU.  MODEL_PATH=/path/to/hub NUM_GENERATIONS=8 ./run_grpo_single_gpu.sh
set -euo pipefail
cd "$(dirname "$0")"
: "${MODEL_PATH:?set MODEL_PATH to a model hub directory}"
ARGS=(--model_path "$MODEL_PATH"
      --data_file "${DATA_FILE:-data/sharegpt_sample.jsonl}"
      --output_dir "${OUTPUT_DIR:-output_grpo}"
      --max_samples "${MAX_SAMPLES:-0}"
      --micro_bsz "${MICRO_BSZ:-2}"
      --num_generations "${NUM_GENERATIONS:-4}"
      --steps_per_generation "${STEPS_PER_GENERATION:-4}"
      --epoch_count "${EPOCHS:-1}"
      --max_prompt_length "${MAX_PROMPT_LENGTH:-1024}"
      --max_completion_length "${MAX_COMPLETION_LENGTH:-256}"
      --temperature "${TEMPERATURE:-0.8}"
      --top_p "${TOP_P:-0.9}"
      --repetition_penalty "${REPETITION_PENALTY:-1.1}"
      --lr_init "${LR_INIT:-1e-6}"
      --lr_final "${LR_FINAL:-1e-7}"
      --warmup_steps "${WARMUP_STEPS:-50}"
      --lora_r "${LORA_R:-64}" --lora_alpha "${LORA_ALPHA:-128}"
      --beta "${BETA:-0.0}"
      --save_every_n_batches "${SAVE_EVERY_N_BATCHES:-0}"
      --save_rollout_steps "${SAVE_ROLLOUT_STEPS:-0}")
[[ -n "${REWARD_WEIGHTS:-}" ]] && ARGS+=(--reward_weights "$REWARD_WEIGHTS")
[[ -n "${SAVE_ROLLOUT_PATH:-}" ]] && ARGS+=(--save_rollout_path "$SAVE_ROLLOUT_PATH")
[[ -n "${ACCELERATOR:-}" ]] && ARGS+=(--accelerator "$ACCELERATOR")      # ACCELERATOR=cpu PRECISION=fp32 runs on the host
[[ -n "${REPORT_TO:-}" ]] && ARGS+=(--report_to "$REPORT_TO" --run_name "${RUN_NAME:-grpo}")
CUDA_VISIBLE_DEVICES="${GPU_ID:-0}" exec python train_grpo_single_gpu.py "${ARGS[@]}"
