"""Where one training step spends its device time, kernel family by kernel family.

    python benchmarks/step_breakdown.py [--layers 4] [--model 1.5b] [--B 8 --T 4096] [--md out.md] [--json out.json]

Builds a model of the named width with ``--layers`` blocks (a few blocks are enough: every block
launches the same kernels), runs warm-up steps, then records ``--steps`` optimiser steps with
``torch.profiler`` (CUPTI kernel records, no replay, no clock change) and sums the device time of
every kernel by name and by family.  The per-block figures scale to the full depth; embedding,
head + loss and the optimiser are reported on their own lines.  The table is the measured split of
a step, which isolated micro-benchmarks cannot give (cache state, clocks under the power cap and
launch gaps differ inside a step).

The reference offers no such tool; its only timing aid is the wall-clock phase monitor of the
GRPO module (``rwkvtune/training/grpo/lightning_module.py:34-107``).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from collections import defaultdict

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

FAMILIES = [
    ("gemm (tcgen05)", r"gemm_tcgen05|splitk_reduce"),
    ("gemm (decode)", r"gemm_decode"),
    ("gemm (library)", r"nvjet|cutlass|cublas|gemm|xmma|sm100_|sm90_"),
    ("wkv7 prep", r"wkv7_tc_prep"),
    ("wkv7 scan fwd", r"wkv7_tc_scan"),
    ("wkv7 scan bwd", r"wkv7_tc_bwd_scan"),
    ("wkv7 chunk bwd", r"wkv7_tc_bwd_chunk"),
    ("wkv7 other", r"wkv7"),
    ("ln_shift_mix fwd", r"ln_shift_mix_fwd|ln_shift_mix_forward"),
    ("ln_shift_mix bwd", r"ln_shift_mix_bwd|ln_shift_mix_backward"),
    ("layer_norm", r"layer_norm|ln_partials"),
    ("timemix_prep fwd", r"timemix_prep_fwd|timemix_prep_forward"),
    ("timemix_prep bwd", r"timemix_prep_bwd|timemix_prep_backward"),
    ("gn_bonus_gate fwd", r"gn_bonus_gate_fwd|gn_bonus_gate_forward"),
    ("gn_bonus_gate bwd", r"gn_bonus_gate_bwd|gn_bonus_gate_backward"),
    ("relu_sq", r"relu_sq"),
    ("ce_rows / logprob rows", r"ce_rows|logprob_entropy"),
    ("embedding / gather", r"embedding|gather_rows"),
    ("optimizer", r"adamw|sumsq|zero2_|p2p_barrier"),
    ("memset / memcpy", r"[Mm]emset|[Mm]emcpy"),
    ("framework element-wise", r"at::native|elementwise|reduce_kernel|vectorized|CatArray|sort|scan"),
]


def family_of(name: str) -> str:
    for fam, pat in FAMILIES:
        if re.search(pat, name):
            return fam
    return "other"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1.5b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--md", default="")
    ap.add_argument("--json", default="")
    a = ap.parse_args()

    import bench
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.parallel import DistContext

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    arch = dict(bench.MODELS[a.model])
    full_layers = arch["n_layer"]
    arch["n_layer"] = a.layers
    cfg = RWKVConfig(vocab_size=65536, ctx_len=a.T, **arch)
    torch.manual_seed(1)
    with torch.device(dev):
        model = RWKV7Model(cfg)
    eng = TrainEngine(model, EngineConfig(lr_init=3e-4, weight_decay=0.01, grad_clip=1.0, precision="bf16", grad_cp=0),
                      DistContext(device=dev))
    ids = torch.randint(0, 65536, (a.B, a.T), device=dev)
    lab = torch.randint(0, 65536, (a.B, a.T), device=dev)
    for _ in range(a.warmup):
        eng.train_step(ids, lab, 3e-4)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        eng.train_step(ids, lab, 3e-4)
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / a.steps

    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(a.steps):
            eng.train_step(ids, lab, 3e-4)
        torch.cuda.synchronize()
    per_kernel = defaultdict(lambda: [0.0, 0])
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        t = getattr(e, "device_time", None)
        if t is None:
            t = e.cuda_time
        per_kernel[e.name][0] += t / 1e3 / a.steps
        per_kernel[e.name][1] += 1
    fam = defaultdict(lambda: [0.0, 0])
    for name, (ms, n) in per_kernel.items():
        f = family_of(name)
        fam[f][0] += ms
        fam[f][1] += n // a.steps
    total = sum(v[0] for v in fam.values())
    lines = [f"model width {a.model}, {a.layers} of {full_layers} blocks, B={a.B}, T={a.T}; "
             f"step {step_ms:.2f} ms by CUDA events (no profiler), kernel time under the profiler {total:.2f} ms",
             "", "| family | ms per step | launches | share |", "|---|---|---|---|"]
    for f, (ms, n) in sorted(fam.items(), key=lambda kv: -kv[1][0]):
        lines.append(f"| {f} | {ms:.3f} | {n} | {100 * ms / total:.1f} % |")
    lines += ["", "| kernel | ms per step | launches per step |", "|---|---|---|"]
    for name, (ms, n) in sorted(per_kernel.items(), key=lambda kv: -kv[1][0])[:40]:
        lines.append(f"| `{name[:100]}` | {ms:.3f} | {n // a.steps} |")
    text = "\n".join(lines)
    print(text)
    if a.md:
        os.makedirs(os.path.dirname(a.md) or ".", exist_ok=True)
        open(a.md, "w").write(text + "\n")
    if a.json:
        os.makedirs(os.path.dirname(a.json) or ".", exist_ok=True)
        json.dump({"step_ms": step_ms, "layers": a.layers, "full_layers": full_layers,
                   "families": {k: v[0] for k, v in fam.items()},
                   "kernels": {k: v for k, v in per_kernel.items()}}, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
