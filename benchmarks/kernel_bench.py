"""Per-kernel micro-benchmarks: CUDA-event timing, achieved GB/s or TFLOP/s, fraction of the measured peak.

    python benchmarks/kernel_bench.py [--only wkv7,ln_shift_mix,...] [--B 8 --T 4096 --C 2048] [--json out.json]

Peaks come from MEASURED_PEAKS.json at the repository root when present (copy bandwidth and
cuBLAS bf16 throughput measured on the same pool), otherwise from the documented fallback
(6650 GB/s, 1590 TFLOP/s).  Inputs are larger than the 126 MB L2 at the default shape.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from rwkvtune_b200 import ops  # noqa: E402

BF = torch.bfloat16


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def bench_wkv7(B, T, C, out):
    from rwkvtune_b200.ops import cuda_ops
    H = C // 64
    r, k, v = (torch.randn(B, T, C, device="cuda").to(BF) for _ in range(3))
    w = (-torch.nn.functional.softplus(-(torch.randn(B, T, C, device="cuda") * 2 - 1)) - 0.5).to(BF)
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, 64, device="cuda"), dim=-1).view(B, T, C)
    a = (-kk).to(BF)
    b = (kk * torch.rand_like(kk)).to(BF)
    ins = [t.requires_grad_(True) for t in (r, w, k, v, a, b)]
    prev = cuda_ops.WKV7_IMPL
    flop = 4 * 2 * B * T * H * 64 * 64
    try:
        for impl in ("simt", "tc"):
            cuda_ops.WKV7_IMPL = impl
            with torch.no_grad():
                ms_inf = timeit(lambda: ops.wkv7(*ins, 64))
            ms_fwd = timeit(lambda: ops.wkv7(*ins, 64))
            y, _ = ops.wkv7(*ins, 64)
            gy = torch.randn_like(y)
            ms_bwd = timeit(lambda: torch.autograd.grad(y, ins, gy, retain_graph=True))
            out[f"wkv7_{impl}_fwd_nograd_ms"] = ms_inf
            out[f"wkv7_{impl}_fwd_train_ms"] = ms_fwd
            out[f"wkv7_{impl}_bwd_ms"] = ms_bwd
            out[f"wkv7_{impl}_fwd_recurrence_tflops"] = flop / ms_inf / 1e9
            del y
    finally:
        cuda_ops.WKV7_IMPL = prev


def bench_elementwise(B, T, C, out, hbm):
    x = torch.randn(B, T, C, device="cuda").to(BF).requires_grad_(True)
    w = torch.ones(C, device="cuda", requires_grad=True)
    b = torch.zeros(C, device="cuda", requires_grad=True)
    nbytes = B * T * C * 2
    for K in (6, 1):
        mix = torch.rand(K, C, device="cuda", requires_grad=True)
        ms = timeit(lambda: ops.ln_shift_mix(x, w, b, mix))
        o, _ = ops.ln_shift_mix(x, w, b, mix)
        go = torch.randn_like(o)
        msb = timeit(lambda: torch.autograd.grad(o, [x, w, b, mix], go, retain_graph=True))
        out[f"ln_shift_mix{K}_fwd_ms"] = ms
        out[f"ln_shift_mix{K}_fwd_frac_hbm"] = (1 + K) * nbytes / ms / 1e6 / hbm
        out[f"ln_shift_mix{K}_bwd_ms"] = msb
        out[f"ln_shift_mix{K}_bwd_frac_hbm"] = (2 + K) * nbytes / msb / 1e6 / hbm
    big = lambda: torch.randn(B, T, C, device="cuda").to(BF).requires_grad_(True)
    par = lambda: torch.randn(1, 1, C, device="cuda", requires_grad=True)
    args = [big(), big(), big(), big(), big(), big(), par(), par(), par(), par(), par()]
    ms = timeit(lambda: ops.timemix_prep(*args, 64))
    outs = ops.timemix_prep(*args, 64)
    gs = [torch.randn_like(o) for o in outs]
    msb = timeit(lambda: torch.autograd.grad(outs, args, gs, retain_graph=True))
    out["timemix_prep_fwd_ms"] = ms
    out["timemix_prep_fwd_frac_hbm"] = 11 * nbytes / ms / 1e6 / hbm
    out["timemix_prep_bwd_ms"] = msb
    out["timemix_prep_bwd_frac_hbm"] = 17 * nbytes / msb / 1e6 / hbm
    args = [big(), big(), big(), big(), big(), torch.ones(C, device="cuda", requires_grad=True),
            torch.zeros(C, device="cuda", requires_grad=True), torch.randn(C // 64, 64, device="cuda", requires_grad=True)]
    ms = timeit(lambda: ops.gn_bonus_gate(*args, 64))
    z = ops.gn_bonus_gate(*args, 64)
    gz = torch.randn_like(z)
    msb = timeit(lambda: torch.autograd.grad(z, args, gz, retain_graph=True))
    out["gn_bonus_gate_fwd_ms"] = ms
    out["gn_bonus_gate_fwd_frac_hbm"] = 6 * nbytes / ms / 1e6 / hbm
    out["gn_bonus_gate_bwd_ms"] = msb
    out["gn_bonus_gate_bwd_frac_hbm"] = 11 * nbytes / msb / 1e6 / hbm


def bench_gemm(B, T, C, out, tf):
    from rwkvtune_b200.ops import gemm
    M = B * T
    for name, (K, N) in {"CxC": (C, C), "Cx4C": (C, 4 * C), "4CxC": (4 * C, C)}.items():
        x = torch.randn(M, K, device="cuda").to(BF)
        w = torch.randn(N, K, device="cuda").to(BF)
        for native in (False, True):
            gemm.set_native(native)
            try:
                ms = timeit(lambda: gemm.mm_nt(x, w))
            finally:
                gemm.set_native(True)
            tag = "native" if native else "cublas"
            out[f"gemm_nt_{name}_{tag}_ms"] = ms
            out[f"gemm_nt_{name}_{tag}_tflops"] = 2 * M * K * N / ms / 1e9
            out[f"gemm_nt_{name}_{tag}_frac_peak"] = 2 * M * K * N / ms / 1e9 / tf
        from rwkvtune_b200.ops import gemm_native
        if hasattr(gemm_native, "mm_nt_2cta"):
            ms = timeit(lambda: gemm_native.mm_nt_2cta(x, w))
            out[f"gemm_nt_{name}_native_2cta_ms"] = ms
            out[f"gemm_nt_{name}_native_2cta_tflops"] = 2 * M * K * N / ms / 1e9
            out[f"gemm_nt_{name}_native_2cta_over_cublas"] = out[f"gemm_nt_{name}_cublas_ms"] / ms
    # weight gradients of the low-rank maps: few output tiles, contraction over every token (split-K)
    for D in (64, 96, 256):
        x = torch.randn(M, C, device="cuda").to(BF)
        h = torch.randn(M, D, device="cuda").to(BF)
        for name, (a, b) in {f"tn_Cx{D}": (x, h), f"tn_{D}xC": (h, x)}.items():
            for native in (False, True):
                gemm.set_native(native)
                try:
                    ms = timeit(lambda: gemm.mm_tn(a, b))
                finally:
                    gemm.set_native(True)
                tag = "native_splitk" if native else "cublas"
                out[f"gemm_{name}_{tag}_us"] = ms * 1e3


def bench_loss(C, out, hbm, M=8192, V=65536):
    """Head + cross-entropy + L2Wrap, forward and backward in one sweep (two 4096-row slabs)."""
    x = (torch.randn(M, C, device="cuda") * 0.5).to(BF).requires_grad_(True)
    w = (torch.randn(V, C, device="cuda") * 0.02).to(BF).requires_grad_(True)
    labels = torch.randint(0, V, (M,), device="cuda")
    ms = timeit(lambda: ops.linear_cross_entropy(x, w, labels, True, -100, M))
    out["linear_ce_fwd_bwd_ms"] = ms
    out["linear_ce_fwd_bwd_tflops"] = 3 * 2 * M * V * C / ms / 1e9
    logits = torch.randn(4096, V, device="cuda").to(BF)
    from rwkvtune_b200.ops._ext import call, f32, i32, i64, ptr, stream
    inv_n = torch.full((1,), 1.0 / 4096, device="cuda")
    rows = torch.empty(4096, device="cuda")
    lab = labels[:4096].contiguous()
    ms = timeit(lambda: call("rwkv_ce_rows", ptr(logits), ptr(lab), ptr(inv_n), f32(1e-8), i64(-100), ptr(rows), i32(1),
                             i64(4096), i32(V), stream()))
    out["ce_rows_slab_ms"] = ms
    out["ce_rows_frac_hbm"] = 2 * logits.numel() * 2 / ms / 1e6 / hbm     # one read (the re-read hits L2) + one write


def _graph_time(fn):
    """Device time of ``fn`` replayed from a CUDA graph (decode steps run from graphs; eager timing of
    microsecond kernels would measure the host)."""
    fn()
    torch.cuda.synchronize()
    from rwkvtune_b200.ops import _ext

    g = torch.cuda.CUDAGraph()
    with _ext.capture_safe_gc(), torch.cuda.graph(g):
        fn()
    return timeit(g.replay)


def bench_decode_gemm(C, out, hbm, M=64):
    """Weight-streaming projections at decode batch sizes: the decode GEMM vs the library GEMM.  Each timed replay
    cycles through enough distinct weight matrices (> L2) that weights come from HBM as in a decode step."""
    from rwkvtune_b200.ops import gemm_native
    for name, (K, N) in {"CxC": (C, C), "Cx4C": (C, 4 * C), "4CxC": (4 * C, C)}.items():
        n_w = max(4, int(256e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device="cuda").to(BF) for _ in range(n_w)]
        x = torch.randn(M, K, device="cuda").to(BF)
        for tag, fn in (("tcgen05_cluster", lambda w: gemm_native.decode_group([x], [w])),
                        ("cublas", lambda w: x @ w.t())):
            ms = _graph_time(lambda: [fn(w) for w in ws]) / n_w
            out[f"decode_gemm_M{M}_{name}_{tag}_us"] = ms * 1e3
            out[f"decode_gemm_M{M}_{name}_{tag}_frac_hbm"] = N * K * 2 / ms / 1e6 / hbm
    ws = [torch.randn(C, C, device="cuda").to(BF) for _ in range(48)]
    xs = [torch.randn(M, C, device="cuda").to(BF) for _ in range(3)]
    ms = _graph_time(lambda: [gemm_native.decode_group(xs, ws[i:i + 3]) for i in range(0, 48, 3)]) / 16
    out[f"decode_gemm_M{M}_3xCxC_tcgen05_cluster_us"] = ms * 1e3
    out[f"decode_gemm_M{M}_3xCxC_tcgen05_cluster_frac_hbm"] = 3 * C * C * 2 / ms / 1e6 / hbm
    ms = _graph_time(lambda: [[x_ @ w.t() for x_, w in zip(xs, ws[i:i + 3])] for i in range(0, 48, 3)]) / 16
    out[f"decode_gemm_M{M}_3xCxC_cublas_us"] = ms * 1e3
    out[f"decode_gemm_M{M}_3xCxC_cublas_frac_hbm"] = 3 * C * C * 2 / ms / 1e6 / hbm


def bench_decode_core(C, out, hbm, paths=64, layers=8):
    """One decoding step of the recurrent core (preparation + WKV7 update + GroupNorm/bonus/gate) as one kernel against
    the three kernels it replaces; `layers` independent state tensors (> L2 together) are walked per timed replay, as
    the layers of a decode step are.  The floor is the state: 2 x paths x H x 64 x 64 x 4 bytes per layer."""
    from rwkvtune_b200 import ops
    from rwkvtune_b200.ops import cuda_ops
    H = C // 64
    bf = lambda s=1.0: (torch.randn(paths, 1, C, device="cuda") * s).to(BF)
    r, k, v, w_lin, a_lin, v_lin, v_first, g = bf(), bf(), bf(), bf(0.5), bf(0.5), bf(0.5), bf(), bf()
    par = lambda s=0.5: torch.nn.Parameter(torch.randn(1, 1, C, device="cuda") * s)
    w0, a0, v0, k_k, k_a = par(), par(), par(), torch.nn.Parameter(par(0.3) + 0.8), torch.nn.Parameter(par(0.3) + 0.8)
    r_k = torch.nn.Parameter(torch.randn(H, 64, device="cuda") * 0.3)
    gn_w = torch.nn.Parameter(1 + 0.1 * torch.randn(C, device="cuda"))
    gn_b = torch.nn.Parameter(0.1 * torch.randn(C, device="cuda"))
    states = [torch.randn(paths, H, 64, 64, device="cuda") * 0.1 for _ in range(layers)]
    floor_bytes = 2 * paths * H * 64 * 64 * 4

    def fused():
        for s in states:
            ops.timemix_decode_core(r, k, v, v_first, w_lin, a_lin, v_lin, g, w0, a0, v0, k_k, k_a, r_k, gn_w, gn_b, s)

    def three():
        for s in states:
            w, k2, v2, a_, b_ = ops.timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, 64)
            ops.wkv7_gn(r, w, k2, v2, a_, b_, g, gn_w, gn_b, r_k, 64, state=s, return_state=True)

    cuda_ops.INPLACE_STATE = True
    try:
        with torch.no_grad():
            for tag, fn in (("fused", fused), ("three_kernels", three)):
                ms = _graph_time(fn) / layers
                out[f"decode_core_{paths}paths_{tag}_us"] = ms * 1e3
                out[f"decode_core_{paths}paths_{tag}_frac_hbm"] = floor_bytes / ms / 1e6 / hbm
    finally:
        cuda_ops.INPLACE_STATE = False


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--C", type=int, default=2048)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    hbm, tf, src = peaks()
    out = {"shape": [a.B, a.T, a.C], "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src}}
    only = set(filter(None, a.only.split(",")))
    if not only or "wkv7" in only:
        bench_wkv7(a.B, a.T, a.C, out)
    if not only or "elementwise" in only:
        bench_elementwise(a.B, a.T, a.C, out, hbm)
    if not only or "gemm" in only:
        bench_gemm(a.B, a.T, a.C, out, tf)
    if not only or "loss" in only:
        bench_loss(a.C, out, hbm)
    if not only or "decode" in only:
        bench_decode_gemm(a.C, out, hbm)
    if not only or "decode_core" in only:
        bench_decode_core(a.C, out, hbm)
    for k, v in out.items():
        print(f"{k}: {v:.4g}" if isinstance(v, float) else f"{k}: {v}")
    if a.json:
        os.makedirs(os.path.dirname(a.json) or ".", exist_ok=True)
        json.dump(out, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
