#!/usr/bin/env python
"""GRPO with LoRA on a ShareGPT role-play file: every assistant turn becomes a prompt, completions are
scored by seven rule-based rewards (``examples/rewards.py``).

    python examples/train_grpo_single_gpu.py --model_path /path/to/hub --data_file chat.jsonl

Flags follow the reference script ``examples/train_grpo_single_gpu.py:414-554``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from rewards import build_reward_functions          # noqa: E402
from sharegpt import build_grpo_dataset, load_sharegpt   # noqa: E402


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model_path", default="models/rwkv7-g1d-0.1b")
    p.add_argument("--data_file", default="data/sharegpt_sample.jsonl")
    p.add_argument("--output_dir", default="output_grpo")
    p.add_argument("--max_samples", type=int, default=0, help="use only the first N prompts (0 = all)")
    p.add_argument("--micro_bsz", type=int, default=2, help="prompts per step")
    p.add_argument("--num_generations", type=int, default=4, help="completions per prompt")
    p.add_argument("--steps_per_generation", type=int, default=4)
    p.add_argument("--epoch_count", type=int, default=1)
    p.add_argument("--max_prompt_length", type=int, default=1024)
    p.add_argument("--max_completion_length", type=int, default=256)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top_p", type=float, default=0.9)
    p.add_argument("--repetition_penalty", type=float, default=1.1)
    p.add_argument("--lr_init", type=float, default=1e-6)
    p.add_argument("--lr_final", type=float, default=1e-7)
    p.add_argument("--warmup_steps", type=int, default=50)
    p.add_argument("--accumulate_grad_batches", type=int, default=1)
    p.add_argument("--precision", default="bf16", choices=["fp32", "fp16", "bf16"])
    p.add_argument("--devices", type=int, default=1)
    p.add_argument("--lora_r", type=int, default=64)
    p.add_argument("--lora_alpha", type=int, default=128)
    p.add_argument("--lora_dropout", type=float, default=0.0)
    p.add_argument("--accelerator", default="gpu", choices=["gpu", "cpu"])
    p.add_argument("--report_to", default="")
    p.add_argument("--run_name", default="rwkvtune-grpo")
    p.add_argument("--reward_weights", default="", help="comma-separated, one per reward function")
    p.add_argument("--beta", type=float, default=0.0, help="KL penalty against the adapter-free model")
    p.add_argument("--advantage_clip", type=float, default=None)
    p.add_argument("--low_reward_threshold", type=float, default=None)
    p.add_argument("--low_reward_scale", type=float, default=0.01)
    p.add_argument("--save_every_n_batches", type=int, default=0)
    p.add_argument("--save_rollout_steps", type=int, default=0)
    p.add_argument("--save_rollout_path", default="")
    return p.parse_args()


def main():
    args = parse_args()
    from rwkvtune_b200 import AutoTokenizer, GRPOConfig, GRPOTrainer, LoraConfig

    tokenizer = AutoTokenizer.from_pretrained(args.model_path)
    dataset = build_grpo_dataset(load_sharegpt(args.data_file), tokenizer, args.max_prompt_length)
    if args.max_samples > 0:
        dataset = dataset[:args.max_samples]
    rewards, weights = build_reward_functions(tokenizer)
    if args.reward_weights:
        weights = [float(w) for w in args.reward_weights.split(",")]
        if len(weights) != len(rewards):
            raise SystemExit(f"--reward_weights has {len(weights)} values for {len(rewards)} reward functions")
    print("[reward]", ", ".join(f"{fn.__name__}={w}" for fn, w in zip(rewards, weights)))

    config = GRPOConfig(
        num_generations=args.num_generations, num_iterations=1, micro_bsz=args.micro_bsz,
        steps_per_generation=args.steps_per_generation, max_prompt_length=args.max_prompt_length,
        max_completion_length=args.max_completion_length, temperature=args.temperature, top_p=args.top_p, top_k=0,
        repetition_penalty=args.repetition_penalty, lr_init=args.lr_init, lr_final=args.lr_final,
        warmup_steps=args.warmup_steps, accumulate_grad_batches=args.accumulate_grad_batches, accelerator=args.accelerator,
        devices=args.devices, precision=args.precision, proj_dir=args.output_dir, epoch_count=args.epoch_count,
        save_every_n_batches=args.save_every_n_batches, save_total_limit=2, report_to=(args.report_to or None),
        run_name=args.run_name, log_steps=1, use_lora=True, reward_weights=weights,
        save_rollout_steps=args.save_rollout_steps, save_rollout_path=(args.save_rollout_path or None),
        beta=args.beta, advantage_clip=args.advantage_clip, low_reward_threshold=args.low_reward_threshold,
        low_reward_scale=args.low_reward_scale)
    peft = LoraConfig(r=args.lora_r, lora_alpha=args.lora_alpha, lora_dropout=args.lora_dropout)
    GRPOTrainer(model=args.model_path, reward_funcs=rewards, args=config, train_dataset=dataset,
                processing_class=tokenizer, peft_config=peft).train()
    print(f"[done] checkpoints under {args.output_dir}")


if __name__ == "__main__":
    main()
