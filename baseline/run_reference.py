"""Reference arm of ``bench.py``: the unmodified reference package from ``baseline/_ref``.

The reference's trainers cannot start offline: ``import rwkvtune`` pulls in ``lightning`` (and
its ZeRO strategies need ``deepspeed``), and neither package exists in the image or the offline
wheelhouse.  What *can* run unmodified is everything the trainers call per step: the reference's
``RWKV7Model`` with its per-block ``torch.utils.checkpoint`` (``grad_cp=1``, the PretrainConfig
default), its own JIT-compiled WKV7 CUDA kernels (``wkv_loader.load_cuda_operator_train``), and its
``CrossEntropyLoss`` + ``L2Wrap`` training-step body.  This runner drives those with the plain
PyTorch pieces Lightning would select for ``precision="bf16"`` on one GPU or ``strategy="ddp"``:
fp32 parameters under bf16 autocast, ``torch.optim.AdamW(fused=True)``, global-norm clipping, and
``DistributedDataParallel`` for N > 1.  A stub ``lightning`` module satisfies the import only; none
of this repository's models, kernels or engine is on the path.  The JSON line says so in
``harness``.
"""
from __future__ import annotations

import json
import os
import sys
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


def _stub_lightning() -> None:
    class _Stub:
        def __init__(self, *a, **k):
            pass

    for name in ("lightning", "lightning.pytorch", "lightning.pytorch.callbacks", "lightning.pytorch.strategies",
                 "lightning.pytorch.loggers", "lightning.pytorch.utilities"):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = []
            sys.modules[name] = mod
    L = sys.modules["lightning"]
    for attr in ("LightningModule", "Trainer", "Callback", "LightningDataModule", "seed_everything"):
        setattr(L, attr, _Stub)
    L.pytorch = sys.modules["lightning.pytorch"]
    for attr in ("LightningModule", "Trainer", "Callback", "seed_everything"):
        setattr(L.pytorch, attr, _Stub)
    for sub in ("callbacks", "strategies", "loggers", "utilities"):
        m = sys.modules[f"lightning.pytorch.{sub}"]
        setattr(L.pytorch, sub, m)
        for attr in ("Callback", "DeepSpeedStrategy", "DDPStrategy", "TensorBoardLogger", "WandbLogger",
                     "rank_zero_only", "rank_zero_info", "ModelCheckpoint"):
            setattr(m, attr, _Stub)


def run_reference(a) -> None:
    if not os.path.isdir(os.path.join(REF, "rwkvtune")):
        return _unavailable("baseline/_ref/rwkvtune is missing (offline install of the reference not present)")
    import torch

    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")
    import torch.distributed as dist

    from bench import MODELS, ClockSampler, vs_baseline

    rank, local_rank, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    os.environ["RWKV_DEVICE"] = "cuda"
    os.environ.setdefault("RWKV_HEAD_SIZE_A", "64")
    sys.path.insert(0, REF)
    _stub_lightning()
    try:
        from rwkvtune.models.configuration import RWKVConfig
        from rwkvtune.models.rwkv7.model import RWKV7Model
        from rwkvtune.models.rwkv7.operators.wkv_loader import load_wkv_operator
        from rwkvtune.training.lightning_module import L2Wrap
    except Exception as exc:
        return _unavailable(f"reference import failed: {type(exc).__name__}: {exc}")
    try:
        load_wkv_operator(device="cuda", for_inference=False, head_size=64)   # JIT build, rank 0 first
    except Exception as exc:
        return _unavailable(f"reference WKV7 kernel build failed: {type(exc).__name__}: {str(exc)[:200]}")

    cfg = RWKVConfig(vocab_size=65536, ctx_len=a.ctx_len, **MODELS[a.model])
    cfg.grad_cp = a.grad_cp
    torch.manual_seed(1234)
    with torch.device(dev):
        model = RWKV7Model(cfg)
    model.train()
    mode = getattr(a, "ref_mode", "autocast")
    if mode == "bf16_master":   # bf16 module + fp32 master weights: the DeepSpeed stage-2 precision regime
        model.to(torch.bfloat16)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], gradient_as_bucket_view=True)
    named = list(model.named_parameters())
    masters = None
    if mode == "bf16_master":
        masters = [torch.nn.Parameter(p.detach().float().clone()) for _, p in named]
        opt_named = [(n, m) for (n, _), m in zip(named, masters)]
    else:
        opt_named = named
    decay = [p for n, p in opt_named if p.ndim >= 2 and ".weight" in n]
    other = [p for n, p in opt_named if not (p.ndim >= 2 and ".weight" in n)]
    opt = torch.optim.AdamW([{"params": other, "weight_decay": 0.0}, {"params": decay, "weight_decay": 0.01}],
                            lr=3e-4, betas=(0.9, 0.99), eps=1e-8, fused=True)
    crit = torch.nn.CrossEntropyLoss(ignore_index=-100)
    B, T, V = a.micro_bsz, a.ctx_len, cfg.vocab_size
    g = torch.Generator().manual_seed(99 + rank)
    n_batches = a.warmup + a.steps
    host_ids = [torch.randint(0, V, (B, T), generator=g).pin_memory() for _ in range(n_batches)]
    host_lab = [torch.randint(0, V, (B, T), generator=g).pin_memory() for _ in range(n_batches)]

    def step(ids, lab):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = net(ids)
            loss = crit(logits.view(-1, logits.size(-1)), lab.view(-1))
            loss = L2Wrap.apply(loss, logits)
        loss.backward()
        if masters is not None:
            for (_, p), m in zip(named, masters):
                m.grad = p.grad.float()
                p.grad = None
            torch.nn.utils.clip_grad_norm_(masters, 1.0)
            opt.step()
            opt.zero_grad(set_to_none=True)
            with torch.no_grad():
                torch._foreach_copy_([p for _, p in named], masters)
            return loss.detach()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    try:
        dev_ids = [t.to(dev) for t in host_ids]
        dev_lab = [t.to(dev) for t in host_lab]
        for i in range(a.warmup):
            step(dev_ids[i], dev_lab[i])
        sampler = ClockSampler(local_rank)
        sync()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.warmup, n_batches):
            loss = step(dev_ids[i], dev_lab[i])
        e1.record()
        sync()
        clocks = sampler.stop()
        ms = e0.elapsed_time(e1)
        final_loss = float(loss)
        sync()
        t0 = time.perf_counter()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        for i in range(a.warmup, n_batches):
            float(step(host_ids[i].to(dev, non_blocking=True), host_lab[i].to(dev, non_blocking=True)))
        e3.record()
        sync()
        ms_e2e = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3)
    except torch.cuda.OutOfMemoryError as exc:
        return _unavailable(f"reference ran out of device memory at this config: {str(exc)[:120]}")

    t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    tokens = B * T * a.steps * world
    value = tokens / (ms / 1e3)
    if rank == 0:
        print(json.dumps({
            "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": vs_baseline(a.model, value, world), "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "final_loss": final_loss,
            "harness": "unmodified reference RWKV7Model + its JIT WKV7 CUDA kernels + CrossEntropy/L2Wrap step body; "
                       + ("bf16 module with fp32 master weights, " if mode == "bf16_master" else "fp32 params under bf16 autocast, ")
                       + "torch AdamW(fused), DDP for N>1 "
                       "(lightning and deepspeed are not installable offline)",
            "config": {"model": f"rwkv7-{a.model}", "global_batch": B * world, "seq_len": T,
                       "parallelism": f"dp{world}", "grad_cp": a.grad_cp},
            "details": {"sharding": "ddp" if world > 1 else "none", "ref_mode": mode},
            "clocks": clocks,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * T * 8,
                    "d2h_bytes_per_step": 4},
        }))
    if world > 1:
        dist.destroy_process_group()
