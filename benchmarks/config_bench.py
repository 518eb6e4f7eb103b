"""Throughput of the other training configurations (the headline pretrain config lives in ``bench.py``).

    python benchmarks/config_bench.py --config lora_zero3   # 2.9B SFT, LoRA r=64, ZeRO-3 when launched on >1 GPU
    python benchmarks/config_bench.py --config infctx       # 0.4B, 65536-token sequences in 4096-token chunks
    python benchmarks/config_bench.py --config grpo         # 1.5B GRPO (dapo, beta 0.04), LoRA r=64, G=8
    python benchmarks/config_bench.py --config collectives  # fused reduce-scatter / AdamW+broadcast vs NVLink roofline
    python benchmarks/config_bench.py --config ag_gemm      # all-gather-fused GEMM vs plain GEMM at the 2.9B shapes
    python benchmarks/config_bench.py --config full_zero3   # full-parameter stage 3 vs stage 2 step time

Multi-GPU: ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/config_bench.py ...``.
Synthetic uniform-random tokens, random-init weights, bf16; timed on the device with CUDA events after warm-up,
max over ranks; prints one JSON line on rank 0.
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

NVLINK_GBS = 770.0           # rate of a plain peer-to-peer copy, per direction per GPU, measured on this machine class
NVLINK_NOMINAL_GBS = 900.0   # NVLink 5: 18 links, per direction per GPU


def _ctx():
    from rwkvtune_b200.parallel import init_distributed

    return init_distributed("gpu")


def _max_over_ranks(ctx, value: float) -> float:
    if ctx.world_size == 1:
        return value
    t = torch.tensor([value], device=ctx.device, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t)


def _time_steps(ctx, step, warmup: int, steps: int) -> float:
    for i in range(warmup):
        step(i)
    if ctx.world_size > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    return _max_over_ranks(ctx, e0.elapsed_time(e1) / steps)


def bench_lora_zero3(a):
    from rwkvtune_b200 import LoraConfig, get_peft_model
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    ctx = _ctx()
    B, T = a.micro_bsz or 2, a.ctx_len or 8192
    cfg = RWKVConfig(vocab_size=65536, ctx_len=T, **MODELS["2.9b"])
    torch.manual_seed(7)
    with torch.device(ctx.device):
        model = RWKV7Model(cfg)
    model = get_peft_model(model, LoraConfig(r=64, lora_alpha=128))
    strategy = "deepspeed_stage_3" if ctx.world_size > 1 else "auto"
    eng = TrainEngine(model, EngineConfig(lr_init=2e-5, grad_clip=1.0, strategy=strategy, precision="bf16", grad_cp=1,
                                          transport="auto"), ctx)
    g = torch.Generator().manual_seed(100 + ctx.rank)
    n = a.warmup + a.steps
    ids = [torch.randint(0, 65536, (B, T), generator=g).to(ctx.device) for _ in range(n)]
    labels = []
    for i in range(n):
        lab = torch.randint(0, 65536, (B, T), generator=g)
        for b in range(B):
            lab[b, :int(torch.randint(128, 2049, (1,), generator=g))] = -100
        labels.append(lab.to(ctx.device))
    state = {"cp": None}

    def step(i):
        eng.train_step(ids[i], labels[i], 2e-5)
        if i == 0:
            torch.cuda.synchronize()
            state["cp"] = eng.autotune_checkpointing(B, T)

    ms = _time_steps(ctx, step, a.warmup, a.steps)
    tokens = B * T * ctx.world_size
    return ctx, {"metric": "train_tokens_per_sec", "value": tokens / ms * 1e3, "ms_per_step": ms,
                 "config": {"model": "rwkv7-2.9b", "lora_r": 64, "seq_len": T, "micro_bsz": B,
                            "parallelism": f"zero3-dp{ctx.world_size}" if ctx.world_size > 1 else "single",
                            "fused_allgather_gemm": eng.zero3 is not None, "checkpointed_layers": state["cp"],
                            "peak_mem_gb": round(eng.phases.peak_bytes() / 2**30, 1)}}


def bench_infctx(a):
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    ctx = _ctx()
    B, T, chunk = a.micro_bsz or 1, a.ctx_len or 65536, 4096
    cfg = RWKVConfig(vocab_size=65536, ctx_len=T, **MODELS["0.4b"])
    torch.manual_seed(7)
    with torch.device(ctx.device):
        model = RWKV7Model(cfg)
    strategy = "deepspeed_stage_2" if ctx.world_size > 1 else "auto"
    eng = TrainEngine(model, EngineConfig(lr_init=1e-4, grad_clip=1.0, strategy=strategy, precision="bf16", grad_cp=1,
                                          train_type="infctx", chunk_ctx=chunk, transport="auto",
                                          cuda_graph=not a.no_graph), ctx)
    g = torch.Generator().manual_seed(100 + ctx.rank)
    n = a.warmup + a.steps
    ids = [torch.randint(0, 65536, (B, T), generator=g).to(ctx.device) for _ in range(n)]
    labels = [torch.randint(0, 65536, (B, T), generator=g).to(ctx.device) for _ in range(n)]
    ms = _time_steps(ctx, lambda i: eng.train_step(ids[i], labels[i], 1e-4), a.warmup, a.steps)
    tokens = B * T * ctx.world_size
    return ctx, {"metric": "train_tokens_per_sec", "value": tokens / ms * 1e3, "ms_per_step": ms,
                 "config": {"model": "rwkv7-0.4b", "seq_len": T, "chunk_ctx": chunk, "micro_bsz": B, "bptt": "truncated",
                            "cuda_graph_chunk_step": not a.no_graph,
                            "parallelism": f"zero2-dp{ctx.world_size}" if ctx.world_size > 1 else "single",
                            "peak_mem_gb": round(eng.phases.peak_bytes() / 2**30, 1)}}


class _IdTokenizer:
    """Text is the space-separated token ids, so a reward function can see ids."""
    eos_token_id = None
    vocab_size = 65536

    def encode(self, text):
        return [int(t) for t in text.split()]

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)


def _low_id_fraction(prompts, completions, **extra):
    out = []
    for c in completions:
        ids = [int(t) for t in c.split()] if c else []
        out.append(sum(i < 32768 for i in ids) / max(1, len(ids)))
    return out


def bench_grpo(a):
    import tempfile

    from rwkvtune_b200 import GRPOConfig, GRPOTrainer, LoraConfig
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    world = int(os.environ.get("WORLD_SIZE", "1"))
    prompts_per_gpu, G, S, P, Cn = a.micro_bsz or 8, 8, 8, 512, a.new_tokens
    cfg = RWKVConfig(vocab_size=65536, ctx_len=4096, eos_token_id=None, **MODELS["1.5b"])
    torch.manual_seed(7)
    model = RWKV7Model(cfg)
    g = torch.Generator().manual_seed(5)
    cycles = 2     # the first rollout + 8 steps warm up (graph capture, allocator); the second is reported
    data = [{"prompt": f"p{i}", "input_ids": torch.randint(1, 65000, (P,), generator=g).tolist()}
            for i in range(prompts_per_gpu * world * cycles)]
    times, rollouts = [], []

    class Clock:
        def on_step_end(self, trainer, metrics):
            torch.cuda.synchronize()
            times.append(time.perf_counter())
            rollouts.append((metrics["rollout/tokens_per_sec"], metrics["rollout/seconds"], metrics["completions/mean_length"]))

    with tempfile.TemporaryDirectory() as tmp:
        args = GRPOConfig(num_generations=G, num_iterations=1, micro_bsz=prompts_per_gpu, steps_per_generation=S,
                          max_prompt_length=P, max_completion_length=Cn, temperature=1.0, top_p=0.95, top_k=0,
                          loss_type="dapo", beta=0.04, lr_init=1e-6, lr_final=1e-7, warmup_steps=0, accelerator="gpu",
                          devices=1, precision="bf16", proj_dir=tmp, epoch_count=1, epoch_steps=S * cycles, use_lora=True,
                          save_total_limit=1, log_steps=1000)
        tr = GRPOTrainer(model=model, reward_funcs=[_low_id_fraction], args=args, train_dataset=data,
                         processing_class=_IdTokenizer(), peft_config=LoraConfig(r=64, lora_alpha=128), callbacks=[Clock()])
        tr.train()
        ctx = tr.ctx
    # second cycle: steps S .. 2S-1; step S includes the rollout, so train time is measured over steps S+1 .. 2S-1
    step_s = (times[2 * S - 1] - times[S]) / (S - 1)
    roll_tps, roll_s, mean_len = rollouts[2 * S - 1]
    seqs_per_step = prompts_per_gpu * G // S
    train_tokens = seqs_per_step * (P + mean_len) * ctx.world_size
    step_s = _max_over_ranks(ctx, step_s)
    roll_s = _max_over_ranks(ctx, roll_s)
    gen_tokens = prompts_per_gpu * G * mean_len * ctx.world_size
    return ctx, {"metric": "grpo_rollout_tokens_per_sec", "value": gen_tokens / roll_s, "rollout_seconds": roll_s,
                 "train_tokens_per_sec": train_tokens / step_s, "train_ms_per_step": step_s * 1e3,
                 "config": {"model": "rwkv7-1.5b", "lora_r": 64, "loss_type": "dapo", "beta": 0.04,
                            "prompts_per_gpu": prompts_per_gpu, "prompt_len": P, "num_generations": G,
                            "max_completion_length": Cn, "steps_per_generation": S, "mean_completion_length": mean_len,
                            "timing": "host clock around device-synchronised steps (through GRPOTrainer.train())",
                            "parallelism": f"dp{ctx.world_size}"}}


def bench_collectives(a):
    """Fused ZeRO-2 kernels on the 1.5B flat parameter space: bytes that must cross NVLink per rank and direction over
    the kernel's time, as a fraction of the link's nominal 900 GB/s and of the 770 GB/s a plain peer copy reaches on
    this pool; then the same kernels inside real training steps, with the bucketed reduce-scatter overlapped with
    backward and without, to show how much communication is left exposed after backward."""
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.ops import _ext

    ctx = _ctx()
    if ctx.world_size < 2:
        raise SystemExit("--config collectives needs at least 2 ranks")
    cfg = RWKVConfig(vocab_size=65536, ctx_len=4096, **MODELS["1.5b"])
    torch.manual_seed(7)
    with torch.device(ctx.device):
        model = RWKV7Model(cfg)
    eng = TrainEngine(model, EngineConfig(lr_init=1e-4, weight_decay=0.01, strategy="deepspeed_stage_2", precision="bf16",
                                          transport="p2p", grad_cp=1), ctx)
    fz, opt, sp = eng.opt._p2p, eng.opt, eng.space
    sp.grads.normal_(0, 1e-3)
    W = ctx.world_size
    shard = opt.hi - opt.lo
    scratch = torch.zeros(1024, dtype=torch.float32, device=ctx.device)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    acc = [0.0, 0.0, 0.0]
    iters = a.warmup + a.steps
    for it in range(iters):
        opt.step_count += 1
        fz._barrier()
        ev[0].record()
        _ext.call("rwkv_zero2_reduce_scatter", fz.grad_ptrs, fz.ctrl_ptrs, _ext.i32(fz.rank), _ext.i32(W), _ext.i64(opt.lo),
                  _ext.i64(shard), _ext.f32(1.0 / W), _ext.ptr(fz.gred), _ext.ptr(scratch), _ext.ptr(fz.status),
                  _ext.stream())
        ev[1].record()
        fz._barrier()
        ev[2].record()
        for gi, s, e in sp.group_segments_in(opt.lo, opt.hi):
            grp = sp.groups[gi]
            lo, hi = s - opt.lo, e - opt.lo
            _ext.call("rwkv_zero2_adam_broadcast", fz.param_ptrs, fz.ctrl_ptrs, _ext.i32(fz.rank), _ext.i32(W), _ext.i64(s),
                      _ext.i64(e - s), _ext.ptr(opt.master[lo:hi]), _ext.ptr(opt.exp_avg[lo:hi]),
                      _ext.ptr(opt.exp_avg_sq[lo:hi]), _ext.ptr(fz.gred[lo:hi]), _ext.f32(1e-6 * grp.lr_scale),
                      _ext.f32(opt.beta1), _ext.f32(opt.beta2), _ext.f32(opt.eps), _ext.f32(grp.weight_decay),
                      _ext.i32(opt.step_count), _ext.f32(opt.grad_clip), _ext.ptr(fz.status), _ext.stream())
        ev[3].record()
        fz._barrier()
        torch.cuda.synchronize()
        if it >= a.warmup:
            acc[0] += ev[0].elapsed_time(ev[1])
            acc[1] += ev[2].elapsed_time(ev[3])
            acc[2] += ev[0].elapsed_time(ev[3])
    fz.check_now()
    rs_ms, ab_ms, all_ms = (_max_over_ranks(ctx, x / a.steps) for x in acc)
    link_bytes = (W - 1) * shard * 2          # bf16 shard pulled from / pushed to each of W-1 peers
    hbm_adam = shard * (3 * 4 * 2 + 4 + 2)     # master, m, v read+write (fp32), reduced grad read, bf16 param write
    rs_gbs, ab_gbs = link_bytes / (rs_ms * 1e-3) / 1e9, link_bytes / (ab_ms * 1e-3) / 1e9

    # ---- inside training steps: time from "backward done" to "parameters published", overlap on and off
    B, T = 8, 4096
    ids = torch.randint(0, 65536, (B, T), device=ctx.device)
    exposed = {}
    for tag, overlap in (("overlap", True), ("serial", False)):
        fz.overlap = overlap
        for _ in range(2):
            eng.train_step(ids, ids, 1e-6)
        fz.timing = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            eng.train_step(ids, ids, 1e-6)
        e1.record()
        torch.cuda.synchronize()
        tail = sum(x.elapsed_time(y) for x, y in fz.timing) / max(len(fz.timing), 1)
        fz.timing = None
        exposed[f"step_ms_{tag}"] = _max_over_ranks(ctx, e0.elapsed_time(e1) / a.steps)
        exposed[f"after_backward_ms_{tag}"] = _max_over_ranks(ctx, tail)
    eng.check_health()
    return ctx, {"metric": "fused_zero2_fraction_of_nvlink_roofline", "value": rs_gbs / NVLINK_NOMINAL_GBS,
                 "reduce_scatter_ms": rs_ms, "reduce_scatter_gbs_in": rs_gbs,
                 "reduce_scatter_frac_of_900_nominal": rs_gbs / NVLINK_NOMINAL_GBS,
                 "reduce_scatter_frac_of_770_measured_peer_copy": rs_gbs / NVLINK_GBS,
                 "adam_broadcast_ms": ab_ms, "adam_broadcast_gbs_out": ab_gbs,
                 "adam_broadcast_frac_of_900_nominal": ab_gbs / NVLINK_NOMINAL_GBS,
                 "adam_broadcast_frac_of_770_measured_peer_copy": ab_gbs / NVLINK_GBS,
                 "adam_broadcast_hbm_floor_ms": hbm_adam / 6548.8e9 * 1e3,
                 "whole_step_ms": all_ms, "link_bytes_per_phase": link_bytes, "adam_hbm_bytes": hbm_adam,
                 "buckets": fz.n_buckets, "reduce_launches_this_rank": len(fz.launch_of_bucket), **exposed,
                 "config": {"model": "rwkv7-1.5b", "elements": int(sp.padded), "shard_elements": int(shard),
                            "parallelism": f"zero2-dp{W}", "global_batch": B * W, "seq_len": T,
                            "roofline": "bytes over NVLink per rank and direction / 900 GB/s nominal; 770 GB/s is the "
                                        "rate of a plain peer-to-peer copy measured on this pool"}}


def bench_ag_gemm(a):
    """The all-gather-fused GEMM in isolation at the 2.9B projection shapes (tokens = 2 x 8192): the fused kernel
    (panels pulled over NVLink by copy CTAs while the MMA CTAs run) against the plain tcgen05 GEMM on a weight that
    is already gathered, and the stand-alone gather kernel.  Roofline: the slower of FLOPs / measured bf16 peak and
    remote panel bytes / link bandwidth."""
    from rwkvtune_b200.ops import gemm_native
    from rwkvtune_b200.parallel.zero3 import Zero3ShardedLinears
    import torch.nn as nn

    ctx = _ctx()
    W = ctx.world_size
    if W < 2:
        raise SystemExit("--config ag_gemm needs at least 2 ranks")
    C, M = 2560, (a.micro_bsz or 2) * (a.ctx_len or 8192)

    class Holder(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([nn.ModuleDict({"att": nn.ModuleDict({"receptance": nn.Linear(C, C, bias=False)}),
                                                        "ffn": nn.ModuleDict({"key": nn.Linear(C, 4 * C, bias=False),
                                                                              "value": nn.Linear(4 * C, C, bias=False)})})
                                         for _ in range(2)])

    torch.manual_seed(3)
    with torch.device(ctx.device):
        holder = Holder().to(torch.bfloat16)
    for p in holder.parameters():
        p.requires_grad_(False)
    full = {n: m.weight.data.clone() for n, m in holder.named_modules() if isinstance(m, nn.Linear)}
    z3 = Zero3ShardedLinears(holder, ctx)
    rows = {}
    peak = 1615.2
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    for sw in z3.sharded:
        if sw.layer != 0:
            continue
        x = torch.randn(M, sw.K, device=ctx.device).to(torch.bfloat16)
        wfull = full[sw.name]
        other = [o for o in z3.sharded if o.slot == sw.slot and o is not sw][0]

        def timed(fn, flush):
            ts = []
            for it in range(a.warmup + a.steps):
                flush()
                if W > 1:
                    torch.distributed.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                if it >= a.warmup:
                    ts.append(e0.elapsed_time(e1))
            ts.sort()
            return _max_over_ranks(ctx, ts[len(ts) // 2])

        nothing = lambda: None
        plain = timed(lambda: gemm_native.mm_nt(x, wfull), nothing)
        fused = timed(lambda: z3.forward_gemm(x, sw), nothing)
        gw = sw.gathered()
        gather = timed(lambda: z3.gather_into(sw, gw, __import__("rwkvtune_b200.ops._ext", fromlist=["x"]).stream()), nothing)
        flops = 2.0 * M * sw.N * sw.K
        remote = sw.N * sw.K * 2 * (W - 1) / W
        floor_ms = max(flops / (peak * 1e12), remote / (NVLINK_NOMINAL_GBS * 1e9)) * 1e3
        y = z3.forward_gemm(x, sw)
        ref = gemm_native.mm_nt(x, wfull)
        rows[sw.slot] = {"N": sw.N, "K": sw.K, "plain_gemm_ms": plain, "fused_ag_gemm_ms": fused, "gather_only_ms": gather,
                         "fused_over_plain": fused / plain, "roofline_floor_ms": floor_ms,
                         "fused_fraction_of_roofline": floor_ms / fused, "remote_bytes": remote,
                         "gather_gbs": remote / (gather * 1e-3) / 1e9,
                         "max_abs_diff_vs_plain": float((y.float() - ref.float()).abs().max())}
        del other
    worst = max(r["fused_over_plain"] for r in rows.values())
    return ctx, {"metric": "ag_gemm_time_over_plain_gemm_time", "value": worst, "shapes": rows,
                 "config": {"model": "rwkv7-2.9b projection shapes", "tokens": M, "parallelism": f"zero3-dp{W}",
                            "roofline": f"max(FLOPs / {peak} TFLOP/s measured, remote panel bytes / 900 GB/s)"}}


def bench_full_zero3(a):
    """Full-parameter training with every projection matrix sharded (stage 3) against the replicated stage-2 run of
    the same model and batch."""
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    ctx = _ctx()
    B, T = a.micro_bsz or 8, a.ctx_len or 4096
    out = {}
    for strategy in ("deepspeed_stage_2", "deepspeed_stage_3"):
        cfg = RWKVConfig(vocab_size=65536, ctx_len=T, **MODELS[a.model or "1.5b"])
        torch.manual_seed(7)
        with torch.device(ctx.device):
            model = RWKV7Model(cfg)
        eng = TrainEngine(model, EngineConfig(lr_init=1e-4, weight_decay=0.01, grad_clip=1.0, strategy=strategy,
                                              precision="bf16", grad_cp=1, transport="p2p"), ctx)
        g = torch.Generator().manual_seed(100 + ctx.rank)
        ids = torch.randint(0, 65536, (B, T), generator=g).to(ctx.device)
        state = {}

        def step(i):
            eng.train_step(ids, ids, 1e-4)
            if i == 0:
                torch.cuda.synchronize()
                state["cp"] = eng.autotune_checkpointing(B, T)

        torch.cuda.reset_peak_memory_stats()
        ms = _time_steps(ctx, step, a.warmup, a.steps)
        eng.check_health()
        out[strategy] = {"ms_per_step": ms, "tokens_per_sec": B * T * ctx.world_size / ms * 1e3,
                         "checkpointed_layers": state.get("cp"),
                         "peak_mem_gb": round(eng.phases.peak_bytes() / 2**30, 1)}
        del eng, model
        torch.cuda.empty_cache()
    s2, s3 = out["deepspeed_stage_2"]["ms_per_step"], out["deepspeed_stage_3"]["ms_per_step"]
    return ctx, {"metric": "zero3_step_time_over_zero2_step_time", "value": s3 / s2, **out,
                 "config": {"model": f"rwkv7-{a.model or '1.5b'}", "seq_len": T, "micro_bsz": B,
                            "parallelism": f"dp{ctx.world_size}"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["lora_zero3", "infctx", "grpo", "collectives", "ag_gemm", "full_zero3"])
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro-bsz", type=int, default=0)
    ap.add_argument("--ctx-len", type=int, default=0)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--model", default="", help="full_zero3: model size (default 1.5b)")
    ap.add_argument("--no-graph", action="store_true", help="infctx: issue every chunk eagerly instead of replaying a CUDA graph")
    a = ap.parse_args()
    ctx, out = {"lora_zero3": bench_lora_zero3, "infctx": bench_infctx, "grpo": bench_grpo,
                "collectives": bench_collectives, "ag_gemm": bench_ag_gemm,
                "full_zero3": bench_full_zero3}[a.config](a)
    out.update({"n_gpus": ctx.world_size, "steps": a.steps, "warmup": a.warmup, "dtype": "bf16", "data": "synthetic"})
    if ctx.is_main:
        print(json.dumps(out))
    if ctx.world_size > 1 and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
