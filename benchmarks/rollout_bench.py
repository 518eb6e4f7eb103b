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
    ap.add_argument("--profile-step", default="", help="write a per-kernel device-time table of ONE decode step "
                                                        "(all layers + head + sampler) to this markdown file")
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
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
                           top_p=0.95, top_k=a.top_k, repetition_penalty=a.repetition_penalty, return_text=False, seed=it)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    tokens = int(out["lengths"].sum())
    print(json.dumps({"metric": "rollout_tokens_per_sec", "value": tokens / dt, "seconds": dt, "generated_tokens": tokens,
                      "paths": a.prompts * a.generations, "prefill_s": gen.last_stats["prefill_s"],
                      "decode_s": gen.last_stats["decode_s"], "cuda_graph": not a.no_graph, "model": a.model}))
    if a.profile_step:
        profile_decode_step(gen, a.prompts * a.generations, a.profile_step)


def profile_decode_step(gen, n: int, path: str) -> None:
    """Device time of every kernel of one decode step at ``n`` paths: the step is issued eagerly (the same kernels the
    CUDA graph replays) under ``torch.profiler`` (CUPTI activity records) together with one sampler launch."""
    from collections import defaultdict

    from torch.profiler import ProfilerActivity, profile

    from rwkvtune_b200.inference import sampling_native
    from rwkvtune_b200.ops import cuda_ops

    dev = gen.device
    state = gen._zero_state(n)
    tok = torch.randint(1, 65000, (n, 1), device=dev)
    cuda_ops.INPLACE_STATE = True
    try:
        with torch.no_grad():
            for _ in range(3):
                logits, _ = gen._forward(tok, state)
                sampling_native.sample_tokens(logits, 1.0, 0.95, seed=1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                e0.record()
                logits, _ = gen._forward(tok, state)
                sampling_native.sample_tokens(logits, 1.0, 0.95, seed=2)
                e1.record()
                torch.cuda.synchronize()
    finally:
        cuda_ops.INPLACE_STATE = False
    agg = defaultdict(lambda: [0.0, 0])
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        t = getattr(e, "device_time", None)
        agg[e.name][0] += (t if t is not None else e.cuda_time)
        agg[e.name][1] += 1
    total = sum(v[0] for v in agg.values())
    lib = sum(v[0] for k, v in agg.items() if any(s in k for s in ("nvjet", "cutlass", "cublas", "gemv", "xmma")))
    lines = [f"one decode step, {n} paths: {sum(v[1] for v in agg.values())} kernels, {total:.0f} us of kernel time "
             f"({lib:.0f} us = {100 * lib / max(total, 1e-9):.0f} % in library GEMM kernels); issued eagerly the step spans "
             f"{e0.elapsed_time(e1) * 1e3:.0f} us on the device", "", "| kernel | us per step | launches |", "|---|---|---|"]
    for name, (us, cnt) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:30]:
        lines.append(f"| `{name[:90]}` | {us:.1f} | {cnt} |")
    text = "\n".join(lines)
    print(text)
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    open(path, "w").write(text + "\n")


if __name__ == "__main__":
    main()
