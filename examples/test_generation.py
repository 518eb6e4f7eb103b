#!/usr/bin/env python
"""Generation smoke test: continue the first user turn of a few ShareGPT samples and print the result next to
the recorded reply.  Optionally loads LoRA weights saved by the trainers (``--lora_path``).

    python examples/test_generation.py --model_path /path/to/hub --data_file chat.jsonl --num_samples 3
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from sharegpt import first_reference, first_user_prompt, load_sharegpt   # noqa: E402


def parse_args():
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model_path", required=True)
    p.add_argument("--lora_path", default=None, help="directory or file with adapter weights")
    p.add_argument("--data_file", default="data/sharegpt_sample.jsonl")
    p.add_argument("--num_samples", type=int, default=3)
    p.add_argument("--max_new_tokens", type=int, default=256)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top_p", type=float, default=0.9)
    p.add_argument("--repetition_penalty", type=float, default=1.0)
    p.add_argument("--eos_token_id", type=int, default=261, help="token that ends a turn (\"\\n\\n\" in the RWKV vocabulary)")
    p.add_argument("--device", default="cuda")
    p.add_argument("--output_json", default="", help="also write prompts / generations / references here")
    return p.parse_args()


def main():
    args = parse_args()
    import torch

    from rwkvtune_b200 import AutoModel, AutoTokenizer
    from rwkvtune_b200.peft import load_peft_model

    tokenizer = AutoTokenizer.from_pretrained(args.model_path)
    model = AutoModel.from_pretrained(args.model_path)
    if args.lora_path:
        model = load_peft_model(model, args.lora_path)
        print(f"[lora] loaded {args.lora_path}")
    dtype = torch.bfloat16 if args.device.startswith("cuda") else torch.float32
    model = model.to(args.device).to(dtype).eval()
    records = [r for r in load_sharegpt(args.data_file) if r.get("conversations")][:args.num_samples]
    eos_text = tokenizer.decode([args.eos_token_id])
    results = []
    for i, rec in enumerate(records, 1):
        prompt = first_user_prompt(rec["conversations"])
        ids = tokenizer.encode(prompt)
        with torch.no_grad():
            out = model.generate(input_ids=torch.tensor([ids], device=args.device),
                                 max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                                 top_p=args.top_p, repetition_penalty=args.repetition_penalty,
                                 eos_token_id=args.eos_token_id)
        new_ids = out[0].tolist()[len(ids):] if hasattr(out, "__getitem__") else list(out)[len(ids):]
        text = tokenizer.decode(new_ids)
        cut = text.find(eos_text) if eos_text else -1
        if cut >= 0:
            text = text[:cut]
        reference = first_reference(rec["conversations"])
        print(f"\n{'-' * 60}\n[sample {i}] {len(ids)} prompt tokens\nPrompt:\n{prompt[-600:]}\n\nGenerated:\n{text}")
        if reference:
            print(f"\nReference:\n{reference}")
        results.append({"prompt": prompt, "generated": text, "reference": reference})
    if args.output_json:
        with open(args.output_json, "w", encoding="utf-8") as f:
            json.dump(results, f, ensure_ascii=False, indent=2)
        print(f"\n[done] wrote {len(results)} records to {args.output_json}")


if __name__ == "__main__":
    main()
