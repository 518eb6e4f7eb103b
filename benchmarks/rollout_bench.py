"""GRPO rollout throughput: prompts x generations decoded in lock-step (by default the 1.5B model, 8 prompts of 512
tokens x 8 generations x 512 new tokens).

    python benchmarks/rollout_bench.py [--model 1.5b] [--prompts 8] [--prompt-len 512] [--generations 8] [--new-tokens 512]

Random-init weights, uniform-random prompt tokens, temperature 1.0, top-p 0.95.  EOS is disabled so every path
decodes exactly ``new-tokens`` tokens; reports generated tokens per second (device-synchronised wall time).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bench import MODELS  # noqa: E402
from rwkvtune_b200.inference import GRPOBatchGenerator  # noqa: E402
from rwkvtune_b200.models import RWKVConfig, RWKV7Model  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1.5b")
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--generations", type=int, default=8)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    cfg = RWKVConfig(vocab_size=65536, ctx_len=8192, eos_token_id=None, **MODELS[a.model])
    with torch.device(dev):
        model = RWKV7Model(cfg)
    model = model.to(torch.bfloat16).eval()
    gen = GRPOBatchGenerator(model, None, dev, eos_token_id=None, use_cuda_graph=not a.no_graph)
    gen.eos_ids = []
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(1, 65000, (a.prompts, a.prompt_len), generator=g).tolist()
    out = None
    for it in range(2):   # first pass builds graphs / warms kernels
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = gen.generate(prompts, max_new_tokens=a.new_tokens, num_generations=a.generations, temperature=1.0,
                           top_p=0.95, return_text=False, seed=it)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    tokens = int(out["lengths"].sum())
    print(json.dumps({"metric": "rollout_tokens_per_sec", "value": tokens / dt, "seconds": dt, "generated_tokens": tokens,
                      "paths": a.prompts * a.generations, "prefill_s": gen.last_stats["prefill_s"],
                      "decode_s": gen.last_stats["decode_s"], "cuda_graph": not a.no_graph, "model": a.model}))


if __name__ == "__main__":
    main()
