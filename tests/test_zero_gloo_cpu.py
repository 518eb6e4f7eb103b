"""Multi-rank host-side logic on CPU (gloo): sharded optimiser against a single process, checkpoints re-sharded
across world sizes, the all-ranks checkpoint veto, and failure detection among real processes."""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
def _free_port() -> int:
    """A port nobody listens on right now (a fixed port can still be held by a rendezvous that has just ended)."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


_RENDEZVOUS_TROUBLE = ("address already in use", "eaddrinuse", "connection refused", "connection reset",
                       "failed to connect", "rendezvous", "socket timeout")


def _launch(script_path, nproc, *args, timeout=420, expect_fail=False):
    env = dict(os.environ, RWKV_ROOT=ROOT, OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    res = None
    for attempt in range(2):
        res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
                              "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script_path),
                              *map(str, args)], capture_output=True, text=True, env=env, timeout=timeout, cwd=ROOT)
        # a port that was free a moment ago can be taken before the launcher binds it: that, and only that, is retried
        trouble = res.returncode != 0 and any(t in (res.stdout + res.stderr).lower() for t in _RENDEZVOUS_TROUBLE)
        if not (trouble and attempt == 0 and not expect_fail):
            break
    if not expect_fail:
        assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res


def _records(stdout):
    """JSON objects printed by the ranks (two ranks may share a line)."""
    import re

    return {r["rank"]: r for r in (json.loads(m) for m in re.findall(r"\{[^{}]*\}", stdout))}


_COMMON = r'''
import os, sys, json, torch
sys.path.insert(0, os.environ["RWKV_ROOT"])
torch.set_num_threads(1)
from rwkvtune_b200.engine import EngineConfig, TrainEngine
from rwkvtune_b200.engine import checkpoint as ckpt
from rwkvtune_b200.models import RWKVConfig, RWKV7Model
from rwkvtune_b200.parallel import init_distributed

def make_engine(ctx, strategy, acc=1):
    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16)
    model = RWKV7Model(cfg)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    return TrainEngine(model, EngineConfig(lr_init=1e-2, weight_decay=0.01, strategy=strategy, precision="fp32",
                                           accumulate_grad_batches=acc), ctx)

def batch(step, rank, B=2, T=16):
    g = torch.Generator().manual_seed(1000 * step + rank)
    idx = torch.randint(0, 128, (B, T), generator=g)
    return idx, idx.roll(-1, 1)
'''

_WORKER_ZERO = _COMMON + r'''
ctx = init_distributed("cpu")
out_dir, world_total = sys.argv[1], int(sys.argv[2])
results = {}
for strategy in ("ddp", "deepspeed_stage_1", "deepspeed_stage_2"):
    eng = make_engine(ctx, strategy)
    for step in range(3):
        if ctx.world_size == 1:     # the single process sees every rank's batch
            pairs = [batch(step, r) for r in range(world_total)]
            idx, lab = torch.cat([p[0] for p in pairs]), torch.cat([p[1] for p in pairs])
        else:
            idx, lab = batch(step, ctx.rank)
        eng.train_step(idx, lab, 1e-2)
    results[strategy] = eng.space.params[:eng.space.numel].clone()
    if ctx.world_size > 1:
        ref = results[strategy].clone()
        torch.distributed.broadcast(ref, 0)
        assert torch.equal(ref, results[strategy]), "ranks hold different parameters after the step"
if ctx.rank == 0:
    torch.save(results, os.path.join(out_dir, f"params_w{ctx.world_size}.pt"))
'''


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_optimizer_matches_single_process(tmp_path, world):
    script = tmp_path / "worker_zero.py"
    script.write_text(_WORKER_ZERO)
    _launch(script, 1, tmp_path, world)
    _launch(script, world, tmp_path, world)
    single = torch.load(tmp_path / "params_w1.pt")
    multi = torch.load(tmp_path / f"params_w{world}.pt")
    for strategy in ("ddp", "deepspeed_stage_1", "deepspeed_stage_2"):
        a, b = single["ddp"], multi[strategy]
        assert torch.allclose(a, b, atol=2e-5, rtol=1e-4), (strategy, (a - b).abs().max())


_WORKER_SAVE = _COMMON + r'''
ctx = init_distributed("cpu")
ck_dir, n_steps = sys.argv[1], int(sys.argv[2])
eng = make_engine(ctx, "deepspeed_stage_2")
for step in range(n_steps):
    eng.train_step(*batch(step, 0), 1e-2)      # every rank the same batch: the trajectory does not depend on W
def write(tmp):
    if ctx.is_main:
        torch.save(eng.model.state_dict(), os.path.join(tmp, "model.pth"))
    ckpt.save_trainer_state(tmp, eng, ctx, {"samples_seen": 0})
ckpt.atomic_checkpoint(ck_dir, ctx, write)
'''

_WORKER_RESUME = _COMMON + r'''
ctx = init_distributed("cpu")
ck_dir, out, first, last = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4])
eng = make_engine(ctx, "deepspeed_stage_2")
if ck_dir != "-":
    sd = torch.load(os.path.join(ck_dir, "model.pth"))
    with torch.no_grad():
        own = eng.model.state_dict()
        for k, v in sd.items():
            own[k].copy_(v)
    assert ckpt.load_optimizer_state(ck_dir, eng, ctx), "optimizer state was not restored"
    assert eng.opt.step_count == first
for step in range(first, last):
    eng.train_step(*batch(step, 0), 1e-2)
if ctx.rank == 0:
    torch.save(eng.space.params[:eng.space.numel].clone(), out)
'''


def test_checkpoint_saved_at_4_ranks_resumes_at_2_and_8(tmp_path):
    save, resume = tmp_path / "save.py", tmp_path / "resume.py"
    save.write_text(_WORKER_SAVE)
    resume.write_text(_WORKER_RESUME)
    ck = tmp_path / "ck"
    _launch(save, 4, ck, 2)
    assert sorted(os.listdir(ck / "trainer_state")) == ["meta.json"] + [f"rank{r}.pt" for r in range(4)]
    _launch(resume, 1, "-", tmp_path / "straight.pt", 0, 4)           # uninterrupted run, one process
    straight = torch.load(tmp_path / "straight.pt")
    for world in (2, 8):
        out = tmp_path / f"resumed_w{world}.pt"
        _launch(resume, world, ck, out, 2, 4)
        got = torch.load(out)
        # fp32 sums in another order per world size: agreement to ~1e-5; a re-sharding error would be orders above
        assert torch.allclose(got, straight, atol=1e-4, rtol=1e-3), (world, (got - straight).abs().max())


def test_missing_shard_is_refused(tmp_path):
    from rwkvtune_b200.engine.checkpoint import check_shards

    shards = [{"world_size": 4, "lo": r * 128, "hi": (r + 1) * 128, "padded": 512} for r in range(4)]
    check_shards(shards)
    with pytest.raises(RuntimeError, match="4 ranks but 3"):
        check_shards(shards[:2] + shards[3:])
    bad = [dict(s) for s in shards]
    bad[2]["lo"] = 300
    with pytest.raises(RuntimeError, match="do not tile"):
        check_shards(bad)


_WORKER_VETO = _COMMON + r'''
ctx = init_distributed("cpu")
ck_dir = sys.argv[1]
eng = make_engine(ctx, "deepspeed_stage_2")
def write_ok(tmp):
    ckpt.save_trainer_state(tmp, eng, ctx, {"generation": 1})
ckpt.atomic_checkpoint(ck_dir, ctx, write_ok)
def write_bad(tmp):
    if ctx.rank == 1:
        raise OSError("no space left on device")
    ckpt.save_trainer_state(tmp, eng, ctx, {"generation": 2})
try:
    ckpt.atomic_checkpoint(ck_dir, ctx, write_bad)
    raised = None
except Exception as exc:
    raised = type(exc).__name__
torch.distributed.barrier()
meta = ckpt.read_meta(ck_dir)
print(json.dumps({"rank": ctx.rank, "raised": raised, "generation": meta.get("generation"),
                  "tmp_left": os.path.exists(ck_dir + ".tmp")}), flush=True)
'''


def test_checkpoint_is_published_only_if_every_rank_wrote(tmp_path):
    script = tmp_path / "veto.py"
    script.write_text(_WORKER_VETO)
    res = _launch(script, 2, tmp_path / "ck")
    recs = _records(res.stdout)
    assert recs[1]["raised"] == "OSError" and recs[0]["raised"] == "RuntimeError"
    assert all(r["generation"] == 1 and not r["tmp_left"] for r in recs.values())   # the old save point survived


_WORKER_GUARD = _COMMON + r'''
import time
from rwkvtune_b200.engine.watchdog import RankFailure, StepAborted
ctx = init_distributed("cpu")
mode, proj = sys.argv[1], sys.argv[2]
eng = make_engine(ctx, "deepspeed_stage_2")
guard = eng.start_guard(timeout_s=2.0)
guard.interval_s = 0.0
guard.hb.interval_s = 0.2
outcome = "finished"
try:
    for step in range(50):
        if mode == "quiet" and step == 2:
            if ctx.rank == 1:
                guard.stop()                   # the rank goes quiet between steps: no collective of its own in flight
                time.sleep(8.0)
                os._exit(0)
            time.sleep(3.5)                    # the survivor is busy on the host for longer than the heartbeat timeout
        if mode == "bad_status" and ctx.rank == 1 and step == 2:
            eng.health_ok = lambda: False      # what an expired device-side wait looks like to the host
        idx, lab = batch(step, ctx.rank)
        guard.before_step()
        eng.train_step(idx, lab, 1e-2)
        guard.after_step(eng.health_ok())
except (RankFailure, StepAborted) as exc:
    outcome = type(exc).__name__ + ":" + str(getattr(exc, "ranks", ""))
    print(json.dumps({"rank": ctx.rank, "outcome": outcome, "step": step}), flush=True)
    os._exit(0)                                # leave without touching the process group again
print(json.dumps({"rank": ctx.rank, "outcome": outcome}), flush=True)
'''


def test_failed_step_stops_all_ranks_together(tmp_path):
    script = tmp_path / "guard.py"
    script.write_text(_WORKER_GUARD)
    res = _launch(script, 2, "bad_status", tmp_path)
    recs = _records(res.stdout)
    assert recs[0]["outcome"].startswith("StepAborted") and recs[1]["outcome"].startswith("StepAborted")
    assert recs[0]["step"] == recs[1]["step"] == 2


def test_quiet_rank_is_noticed_on_the_host_before_the_next_launch(tmp_path):
    script = tmp_path / "guard.py"
    script.write_text(_WORKER_GUARD)
    res = _launch(script, 2, "quiet", tmp_path, expect_fail=True)
    recs = _records(res.stdout)
    assert recs[0]["outcome"] == "RankFailure:[1]" and recs[0]["step"] == 2, res.stdout[-2000:] + res.stderr[-2000:]


def test_emergency_save_is_written_by_the_lowest_live_rank(tmp_path):
    from rwkvtune_b200 import SFTConfig, SFTTrainer
    from rwkvtune_b200.engine.watchdog import RankFailure
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.parallel import DistContext

    torch.manual_seed(0)
    model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16))
    data = [{"input_ids": [1, 2, 3, 4], "labels": [2, 3, 4, 5]}] * 4
    for rank, dead, writes in ((1, [0], True), (1, [2], False), (0, [2], True)):
        proj = tmp_path / f"p{rank}{dead[0]}"
        tr = SFTTrainer(model, SFTConfig(ctx_len=16, micro_bsz=1, accelerator="cpu", precision="fp32", proj_dir=str(proj)), data)
        tr.ctx = DistContext(rank=rank, world_size=3)
        tr._emergency_save(RankFailure(dead))
        assert os.path.exists(proj / "rwkv7-emergency" / "model.pth") == writes
    tr._emergency_save(ValueError("not a distributed failure"))      # other errors do not trigger a save
