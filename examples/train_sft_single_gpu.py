#!/usr/bin/env python
"""Supervised fine-tuning of an RWKV-7 model hub on a ShareGPT file, on one GPU.

    python examples/train_sft_single_gpu.py --model_path /path/to/hub --data_file chat.jsonl --use_lora

Same flags as the reference script ``examples/train_sft_single_gpu.py:273-338``; the model hub is the directory
written by ``rwkvtune-create-hub`` (``config.json``, ``model.pth``, tokenizer files).
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from sharegpt import IGNORE_INDEX, build_sft_dataset, load_sharegpt   # noqa: E402


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model_path", required=True, help="model hub directory")
    p.add_argument("--data_file", default="data/sharegpt_sample.jsonl", help="ShareGPT .jsonl / .json")
    p.add_argument("--ctx_len", type=int, default=2048)
    p.add_argument("--last_reply_only", action="store_true", help="learn only the final assistant turn of each sample")
    p.add_argument("--micro_bsz", type=int, default=2)
    p.add_argument("--accumulate_grad_batches", type=int, default=4)
    p.add_argument("--epoch_count", type=int, default=3)
    p.add_argument("--lr_init", type=float, default=2e-5)
    p.add_argument("--lr_final", type=float, default=1e-6)
    p.add_argument("--warmup_steps", type=int, default=10)
    p.add_argument("--use_lora", action="store_true")
    p.add_argument("--lora_r", type=int, default=64)
    p.add_argument("--lora_alpha", type=int, default=128)
    p.add_argument("--lora_dropout", type=float, default=0.0)
    p.add_argument("--output_dir", default="output_sft")
    p.add_argument("--epoch_save", type=int, default=1)
    p.add_argument("--save_total_limit", type=int, default=3)
    p.add_argument("--precision", default="bf16", choices=["fp32", "fp16", "bf16"])
    p.add_argument("--accelerator", default="gpu", choices=["gpu", "cpu"])
    p.add_argument("--report_to", default="")
    p.add_argument("--run_name", default="")
    p.add_argument("--log_every_n_steps", type=int, default=1)
    return p.parse_args()


def show_sample(sample, tokenizer, limit: int = 400):
    learned = [t for t in sample["labels"] if t != IGNORE_INDEX]
    print(f"[data] first sample: {len(sample['input_ids'])} tokens, {len(learned)} with loss")
    print("[data] input :", repr(tokenizer.decode(sample["input_ids"])[:limit]))
    print("[data] target:", repr(tokenizer.decode(learned)[:limit]))


def main():
    args = parse_args()
    from rwkvtune_b200 import AutoModel, AutoTokenizer, LoraConfig, SFTConfig, SFTTrainer, get_peft_model

    tokenizer = AutoTokenizer.from_pretrained(args.model_path)
    eos = getattr(tokenizer, "eos_token_id", None)
    print(f"[tokenizer] vocab {tokenizer.vocab_size}, eos {eos}")
    dataset = build_sft_dataset(load_sharegpt(args.data_file), tokenizer, args.ctx_len, args.last_reply_only, eos)
    show_sample(dataset[0], tokenizer)

    model = AutoModel.from_pretrained(args.model_path)
    cfg = model.config
    print(f"[model] {cfg.n_layer} layers, n_embd {cfg.n_embd}, vocab {cfg.vocab_size}")
    lora = None
    if args.use_lora:
        lora = {"r": args.lora_r, "lora_alpha": args.lora_alpha, "lora_dropout": args.lora_dropout}
        model = get_peft_model(model, LoraConfig(**lora))
        n_train = sum(p.numel() for p in model.parameters() if p.requires_grad)
        n_all = sum(p.numel() for p in model.parameters())
        print(f"[lora] r={args.lora_r}: {n_train:,} of {n_all:,} parameters train ({100 * n_train / n_all:.2f}%)")

    config = SFTConfig(ctx_len=args.ctx_len, micro_bsz=args.micro_bsz,
                       accumulate_grad_batches=args.accumulate_grad_batches, epoch_count=args.epoch_count,
                       epoch_save=args.epoch_save, save_total_limit=args.save_total_limit, lr_init=args.lr_init,
                       lr_final=args.lr_final, warmup_steps=args.warmup_steps, devices=1, accelerator=args.accelerator, precision=args.precision,
                       proj_dir=args.output_dir, use_lora=args.use_lora,
                       lora_save_mode="lora_only" if args.use_lora else "full", report_to=args.report_to,
                       run_name=args.run_name, log_every_n_steps=args.log_every_n_steps)
    print(f"[train] ctx {config.ctx_len}, batch {config.micro_bsz} x accum {config.accumulate_grad_batches}, "
          f"{config.epoch_count} epochs, lr {config.lr_init} -> {config.lr_final}, {config.precision}")
    SFTTrainer(model=model, args=config, train_dataset=dataset, processing_class=tokenizer, lora_config=lora).train()
    print(f"[done] checkpoints under {args.output_dir}")


if __name__ == "__main__":
    main()
