"""The trainers at two CPU ranks (gloo): sharded optimiser through ``SFTTrainer`` with a save point that a single
process resumes, and ``GRPOTrainer`` with prompts split by rank and reward statistics taken over the whole job."""
import json
import os
import re
import socket
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(script, nproc, *args, timeout=420):
    env = dict(os.environ, RWKV_ROOT=ROOT, OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(script), *map(str, args)]
    if nproc == 1:
        cmd = [sys.executable, str(script), *map(str, args)]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout, cwd=ROOT)
    trouble = ("address already in use", "eaddrinuse", "connection refused", "failed to connect", "socket timeout")
    if res.returncode != 0 and nproc > 1 and any(t in (res.stdout + res.stderr).lower() for t in trouble):
        # the port that was free a moment ago was taken before the launcher bound it: once more on another one
        cmd[cmd.index("--master-port") + 1] = str(_free_port())
        res = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=timeout, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    # two ranks can share an output line: pick the flat JSON objects out, wherever they sit
    return [json.loads(m) for m in re.findall(r"REC (\{[^{}]*\})", res.stdout)]


_PRELUDE = r'''
import os, sys, json, torch
sys.path.insert(0, os.environ["RWKV_ROOT"])
torch.set_num_threads(1)
from rwkvtune_b200.models import RWKVConfig, RWKV7Model

def make_model(**kw):
    torch.manual_seed(0)
    m = RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16, **kw))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    return m
'''

_SFT = _PRELUDE + r'''
from rwkvtune_b200 import SFTConfig, SFTTrainer
proj, epochs, resume = sys.argv[1], int(sys.argv[2]), sys.argv[3]
g = torch.Generator().manual_seed(0)
base = torch.randint(1, 128, (4, 33), generator=g)
rows = [{"input_ids": base[i % 4][:-1].tolist(), "labels": base[i % 4][1:].tolist()} for i in range(16)]
world = int(os.environ.get("WORLD_SIZE", "1"))
args = SFTConfig(ctx_len=32, micro_bsz=4 // world, epoch_count=epochs, lr_init=3e-3, lr_final=1e-3, warmup_steps=0,
                 accelerator="cpu", devices=world, strategy="deepspeed_stage_2", precision="fp32", proj_dir=proj, grad_cp=0,
                 epoch_save=1, save_total_limit=0, dataloader_shuffle=False,
                 resume_from_checkpoint=(None if resume == "-" else resume))
tr = SFTTrainer(make_model(), args, rows)
tr.train()
print("REC " + json.dumps({"rank": tr.ctx.rank, "world": tr.ctx.world_size, "samples_seen": tr.state["samples_seen"],
                           "owned": [int(tr.engine.opt.lo), int(tr.engine.opt.hi)]}), flush=True)
'''


def _losses(proj):
    return [json.loads(l)["loss"] for l in open(os.path.join(proj, "loss_data.jsonl"))]


def test_sft_trainer_at_two_ranks_shards_the_optimizer_and_one_process_resumes(tmp_path):
    script = tmp_path / "sft.py"
    script.write_text(_SFT)
    two = tmp_path / "two"
    recs = _launch(script, 2, two, 2, "-")
    assert sorted(r["rank"] for r in recs) == [0, 1] and all(r["world"] == 2 and r["samples_seen"] == 32 for r in recs)
    owned = sorted(r["owned"] for r in recs)
    assert owned[0][0] == 0 and owned[0][1] == owned[1][0] and owned[1][1] > owned[1][0]      # two ranges that tile
    ck = two / "rwkv7-epoch1"
    assert sorted(os.listdir(ck / "trainer_state")) == ["meta.json", "rank0.pt", "rank1.pt"]
    assert json.load(open(ck / "trainer_state" / "meta.json"))["devices"] == 2
    # the same global batches in one process (4 samples per step either way): same loss curve ...
    one = tmp_path / "one"
    _launch(script, 1, one, 2, "-")
    a, b = _losses(str(two)), _losses(str(one))
    assert len(a) == len(b) == 8 and all(abs(x - y) < 2e-4 for x, y in zip(a, b)), (a, b)
    # ... and one process picks up the two-rank save point (optimiser shards merged) and continues that curve
    resumed = tmp_path / "resumed"
    recs = _launch(script, 1, resumed, 2, ck)
    assert recs[0]["world"] == 1 and recs[0]["samples_seen"] == 32
    tail = _losses(str(resumed))
    assert len(tail) == 4 and all(abs(x - y) < 2e-4 for x, y in zip(a[4:], tail)), (a[4:], tail)


_GRPO = _PRELUDE + r'''
from rwkvtune_b200 import GRPOConfig, GRPOTrainer, LoraConfig
proj = sys.argv[1]

class Tok:
    eos_token_id = 7
    pad_token_id = 0
    vocab_size = 128
    def encode(self, s): return [8 + ord(c) % 100 for c in s]
    def decode(self, ids, **kw): return " ".join(str(int(i)) for i in ids)
    def save_pretrained(self, d): pass

seen = []
def by_prompt(prompts, completions, tag, **kw):          # depends on which prompts this rank was given
    seen.extend(tag)
    return [float(t) for t in tag]
def by_length(prompts, completions, **kw):
    return [len(c.split()) / 10.0 for c in completions]

data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i, 12 + i], "tag": i} for i in range(8)]
world = int(os.environ.get("WORLD_SIZE", "1"))
args = GRPOConfig(micro_bsz=2, num_generations=2, steps_per_generation=1, max_prompt_length=8, max_completion_length=4,
                  beta=0.0, lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="cpu", devices=world, precision="fp32",
                  proj_dir=proj, epoch_count=1, epoch_steps=1, log_steps=1, scale_rewards="batch")
tr = GRPOTrainer(make_model(eos_token_id=7), [by_prompt, by_length], args, data, processing_class=Tok(),
                 peft_config=LoraConfig(r=4, lora_alpha=8))
tr.train()
m = tr.last_metrics
print("REC " + json.dumps({"rank": tr.ctx.rank, "tags": sorted(set(seen)), "local_mean": sum(seen) / len(seen),
                           "job_mean": m["train/rewards/by_prompt/mean"], "job_min": m["train/rewards/by_prompt/min"],
                           "job_max": m["train/rewards/by_prompt/max"], "reward_mean": m["train/reward/mean"],
                           "len_mean": m["train/rewards/by_length/mean"]}), flush=True)
'''


def test_grpo_trainer_at_two_ranks_splits_prompts_and_reports_job_wide_rewards(tmp_path):
    script = tmp_path / "grpo.py"
    script.write_text(_GRPO)
    recs = sorted(_launch(script, 2, tmp_path / "g"), key=lambda r: r["rank"])
    assert len(recs) == 2
    t0, t1 = set(recs[0]["tags"]), set(recs[1]["tags"])
    assert t0 and t1 and not (t0 & t1), (t0, t1)                       # each rank rolled out its own prompts
    # both ranks log the same statistics, and they are those of all rewards of the job, not of the local ones
    for key in ("job_mean", "job_min", "job_max", "reward_mean", "len_mean"):
        assert abs(recs[0][key] - recs[1][key]) < 1e-6, key
    want = (recs[0]["local_mean"] + recs[1]["local_mean"]) / 2
    assert abs(recs[0]["job_mean"] - want) < 1e-6
    assert recs[0]["job_min"] == min(t0 | t1) and recs[0]["job_max"] == max(t0 | t1)
    assert recs[0]["local_mean"] != recs[1]["local_mean"]
