"""Where the time of one decode GEMM launch goes: per-CTA phase stamps (``%globaltimer``) written by the kernel itself.

    python benchmarks/decode_gemm_timeline.py [--M 64] [--C 2048]

For each of the three projection shapes of a block (C x C, C -> 4C, 4C -> C) one launch is traced with the weights
evicted from L2 (a 256 MB fill in between), and the minimum / median / maximum over the CTAs of every phase is
printed in microseconds after the first CTA started.  The stamps cost a predicated store each; the launch is
otherwise the production kernel (``rwkvtune_b200/csrc/gemm_decode_tcgen05.cu``).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

PHASES = ["CTA started", "barriers armed, tensor memory allocated", "chain wait returned", "first ring stage landed",
          "last ring stage landed", "accumulator complete", "partial tile in shared memory", "cluster barrier passed",
          "rows summed and stored", "tensor memory released"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=64)
    ap.add_argument("--C", type=int, default=2048)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    from rwkvtune_b200.ops import gemm_native

    BF = torch.bfloat16
    C, M = a.C, a.M
    lines = []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name, (N, K) in {"CxC": (C, C), "C->4C": (4 * C, C), "4C->C": (C, 4 * C)}.items():
        w = (torch.randn(N, K, device="cuda") * 0.05).to(BF)
        x = torch.randn(M, K, device="cuda").to(BF)
        for _ in range(3):
            gemm_native.decode_group([x], [w])
        trace = torch.zeros(4096 * 16, dtype=torch.int64, device="cuda")
        flush.zero_()
        torch.cuda.synchronize()
        (y,) = gemm_native.decode_group([x], [w], trace=trace)
        torch.cuda.synchronize()
        t = trace.view(-1, 16).cpu()
        t = t[t[:, 0] > 0]
        t0 = int(t[:, 0].min())
        err = (y.float() - x.float() @ w.float().t()).abs().max().item()
        lines.append(f"### {name}: x [{M}, {K}] @ W [{N}, {K}]^T, {t.shape[0]} CTAs, {N * K * 2 / 1e6:.1f} MB of weights "
                     f"(max abs error {err:.3f})")
        lines.append("")
        lines.append("| phase | min us | median us | max us |")
        lines.append("|---|---|---|---|")
        for i, ph in enumerate(PHASES):
            col = t[:, i][t[:, i] > 0]
            if col.numel():
                rel = (col - t0).double() / 1e3
                lines.append(f"| {ph} | {rel.min():.2f} | {rel.median():.2f} | {rel.max():.2f} |")
        lines.append("")
    text = "\n".join(lines)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")


if __name__ == "__main__":
    main()
