"""RWKV-7 0.1B fp32 SFT step on the host CPU (pure-PyTorch WKV7 recurrence), both arms.

    python benchmarks/cpu_sft_bench.py                    # this package: TrainEngine on CPU, fp32
    python benchmarks/cpu_sft_bench.py --impl reference   # the unmodified reference model, CPU operator and L2Wrap

Shape: L=12, D=768, vocabulary 65536, random init, micro-batch 2 x 256 tokens, ids uniform in [0, 65536), labels =
ids shifted by one with the first 64 positions of every row set to -100, AdamW (lr 2e-5), cross-entropy + L2Wrap,
gradient clipping at 1.0.  Prints one JSON line with seconds per step (median of the timed steps) and tokens/s.
The reference arm drives the reference's own ``RWKV7Model`` (``rwkvtune/models/rwkv7/model.py:421-466``), its CPU
operator (``operators/wkv_cpu.py:9-80``, selected with ``RWKV_DEVICE=cpu``) and its ``L2Wrap``
(``training/lightning_module.py:23-39``) with ``torch.optim.AdamW``; ``lightning`` is replaced by an import stub.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

B, T, V, MASKED = 2, 256, 65536, 64


def batch(step: int):
    g = torch.Generator().manual_seed(1234 + step)
    ids = torch.randint(0, V, (B, T + 1), generator=g)
    labels = ids[:, 1:].clone()
    labels[:, :MASKED] = -100
    return ids[:, :-1].contiguous(), labels


def run_ours(steps: int, warmup: int):
    from rwkvtune_b200.configs import load_model_config
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKV7Model
    from rwkvtune_b200.parallel import DistContext

    torch.manual_seed(0)
    model = RWKV7Model(load_model_config("0.1b").to_rwkv_config())
    eng = TrainEngine(model, EngineConfig(lr_init=2e-5, precision="fp32", grad_clip=1.0, grad_cp=0), DistContext())
    times, losses = [], []
    for s in range(warmup + steps):
        ids, labels = batch(s)
        t0 = time.perf_counter()
        loss = eng.train_step_from_host(ids, labels, 2e-5)
        dt = time.perf_counter() - t0
        if s >= warmup:
            times.append(dt)
        losses.append(float(loss))
    return times, losses


def run_reference(steps: int, warmup: int):
    from baseline.run_reference import REF, _stub_lightning

    if not os.path.isdir(os.path.join(REF, "rwkvtune")):
        return None, None
    os.environ["RWKV_DEVICE"] = "cpu"
    sys.path.insert(0, REF)
    _stub_lightning()
    from rwkvtune.models.configuration import RWKVConfig
    from rwkvtune.models.rwkv7.model import RWKV7Model
    from rwkvtune.training.lightning_module import L2Wrap

    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=12, n_embd=768, vocab_size=V, head_size_a=64, ctx_len=4096, dim_att_lora=64, dim_gate_lora=128,
                     dim_mv_lora=32)
    model = RWKV7Model(cfg).float()
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.0)
    ce = torch.nn.CrossEntropyLoss(ignore_index=-100)
    times, losses = [], []
    for s in range(warmup + steps):
        ids, labels = batch(s)
        t0 = time.perf_counter()
        logits = model(ids)
        loss = L2Wrap.apply(ce(logits.view(-1, logits.size(-1)), labels.view(-1)), logits)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        dt = time.perf_counter() - t0
        if s >= warmup:
            times.append(dt)
        losses.append(float(loss))
    return times, losses


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    a = ap.parse_args()
    times, losses = (run_ours if a.impl == "ours" else run_reference)(a.steps, a.warmup)
    if times is None:
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/rwkvtune is missing"}))
        return
    med = statistics.median(times)
    print(json.dumps({"impl": a.impl, "metric": "cpu_sft_step_seconds", "value": round(med, 3), "tokens_per_s": round(B * T / med, 1),
                      "min_s": round(min(times), 3), "max_s": round(max(times), 3), "steps": a.steps, "warmup": a.warmup,
                      "first_loss": round(losses[0], 4), "last_loss": round(losses[-1], 4), "threads": torch.get_num_threads(),
                      "config": {"model": "rwkv7-0.1b", "micro_bsz": B, "ctx_len": T, "dtype": "fp32", "device": "cpu"}}))


if __name__ == "__main__":
    main()
