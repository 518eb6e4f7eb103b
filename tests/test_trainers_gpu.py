"""The trainers end to end on one GPU through the public API (bf16, native kernels): supervised full-parameter and
LoRA runs with their save points, and a GRPO run (rollout engine + policy step)."""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(**kw):
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=256, vocab_size=512, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32, **kw)
    m = RWKV7Model(cfg)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.02)
    return m


def _dataset(n=32, T=64, V=512):
    g = torch.Generator().manual_seed(0)
    base = torch.randint(1, V, (4, T + 1), generator=g)
    rows = []
    for i in range(n):
        row = base[i % 4]
        labels = row[1:].clone()
        labels[:4] = -100
        rows.append({"input_ids": row[:-1].tolist(), "labels": labels.tolist()})
    return rows


def _losses(proj, name="loss_data.jsonl"):
    return [json.loads(l)["loss"] for l in open(os.path.join(proj, name))]


def test_sft_on_gpu_learns_saves_and_reloads(tmp_path):
    from rwkvtune_b200 import AutoModel, SFTConfig, SFTTrainer
    from rwkvtune_b200.ops import _ext

    proj = str(tmp_path / "sft")
    args = SFTConfig(ctx_len=64, micro_bsz=4, epoch_count=3, lr_init=3e-3, lr_final=1e-3, warmup_steps=2,
                     accelerator="gpu", devices=1, precision="bf16", proj_dir=proj, grad_cp=0)
    seen = []

    class Probe:
        def on_train_batch_end(self, trainer, outputs, batch, batch_idx):
            seen.append(outputs["loss"])

    before = _ext.launch_count()
    tr = SFTTrainer(_model(), args, _dataset(), callbacks=[Probe()])
    tr.train()
    assert _ext.launch_count() > before, "the run did not go through the native kernels"
    losses = _losses(proj)
    assert len(losses) == len(seen) == 24 and losses[-1] < losses[0] - 0.5, (losses[0], losses[-1])
    ck = os.path.join(proj, "rwkv7-epoch3")
    assert {"config.json", "model.pth", "trainer_state"} <= set(os.listdir(ck))
    reloaded = AutoModel.from_pretrained(ck, device="cuda", dtype=torch.bfloat16).eval()
    idx = torch.tensor([_dataset()[0]["input_ids"]], device="cuda")
    with torch.no_grad():
        a, b = reloaded(idx).float(), tr.model(idx).float()
    assert float((a - b).abs().max()) < 0.05 + 0.02 * float(b.abs().max())


def test_lora_sft_on_gpu_trains_adapters_only_and_merges(tmp_path):
    from rwkvtune_b200 import AutoModel, LoraConfig, SFTConfig, SFTTrainer, load_peft_model

    proj = str(tmp_path / "lora")
    base = _model()
    frozen = {n: p.detach().clone() for n, p in base.named_parameters() if n.endswith("att.key.weight")}
    args = SFTConfig(ctx_len=64, micro_bsz=4, epoch_count=3, lr_init=5e-3, lr_final=1e-3, warmup_steps=2,
                     accelerator="gpu", devices=1, precision="bf16", proj_dir=proj, grad_cp=0, lora_save_mode="both")
    tr = SFTTrainer(base, args, _dataset(), lora_config=LoraConfig(r=16, lora_alpha=32))
    tr.train()
    losses = _losses(proj)
    assert losses[-1] < losses[0] - 0.3, (losses[0], losses[-1])
    checked = 0
    for n, p in tr.model.named_parameters():
        if n.endswith("att.key.base_layer.weight"):
            assert torch.equal(p.detach().float().cpu(), frozen[n.replace(".base_layer", "")].to(p.dtype).float())
            checked += 1
    assert checked == 2, "base weights of the adapted layers were not found"
    ck = os.path.join(proj, "rwkv7-epoch3")
    files = set(os.listdir(ck))
    assert {"adapter_model.bin", "adapter_config.json", "merged"} <= files, files
    merged = AutoModel.from_pretrained(os.path.join(ck, "merged"), device="cuda", dtype=torch.bfloat16).eval()
    idx = torch.tensor([_dataset()[1]["input_ids"]], device="cuda")
    with torch.no_grad():
        want = tr.model(idx).float()
        got = merged(idx).float()
    assert float((got - want).abs().max()) < 0.1 + 0.05 * float(want.abs().max())      # merged weights are re-rounded to bf16


class _Tok:
    eos_token_id = 7
    pad_token_id = 0
    vocab_size = 512

    def encode(self, s):
        return [8 + (ord(c) % 200) for c in s]

    def decode(self, ids, **kw):
        return " ".join(str(int(i)) for i in ids)

    def save_pretrained(self, d):
        pass


def test_grpo_on_gpu_rolls_out_and_steps(tmp_path):
    from rwkvtune_b200 import GRPOConfig, GRPOTrainer, LoraConfig

    proj = str(tmp_path / "grpo")
    data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i, 12 + i, 13 + i]} for i in range(4)]
    args = GRPOConfig(micro_bsz=2, num_generations=4, steps_per_generation=2, max_prompt_length=8, max_completion_length=16,
                      temperature=1.0, top_p=0.95, beta=0.04, lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="gpu",
                      devices=1, precision="bf16", proj_dir=proj, epoch_count=1, log_steps=1)

    def reward(prompts, completions, **kw):       # prefers small token ids: dense, varies inside a group
        return [-sum(int(t) for t in c.split()) / (1 + len(c.split())) / 512 for c in completions]

    tr = GRPOTrainer(_model(eos_token_id=7), reward, args, data, processing_class=_Tok(),
                     peft_config=LoraConfig(r=8, lora_alpha=16))
    tr.train()
    recs = [json.loads(l) for l in open(os.path.join(proj, "grpo_loss_data.jsonl"))]
    assert len(recs) == 4
    m = tr.last_metrics
    for key in ("train_loss", "kl_div", "entropy", "train/reward/mean", "completions/mean_length"):
        assert key in m and m[key] == m[key], key
    assert m["completions/mean_length"] > 0 and m["kl_div"] > -1e-3
    moved = any(float(p.detach().abs().sum()) > 0 for n, p in tr.engine.model.named_parameters() if "lora_B" in n)
    assert moved, "adapters never received an update"
    assert {"adapter_model.bin", "trainer_state"} <= set(os.listdir(os.path.join(proj, "checkpoint_epoch_1")))


@pytest.mark.parametrize("truncated", [True, False])
def test_pretrain_infctx_on_gpu_from_an_iterable(tmp_path, truncated):
    from rwkvtune_b200 import PretrainConfig, PretrainTrainer

    class Stream:
        def __iter__(self):
            return iter(_dataset(24, T=128))

    proj = str(tmp_path / "pre")
    args = PretrainConfig(ctx_len=128, micro_bsz=2, epoch_count=1, epoch_steps=10, train_type="infctx", chunk_ctx=32,
                          truncated_bptt=truncated, lr_init=3e-3, warmup_steps=0, accelerator="gpu", devices=1,
                          precision="bf16", proj_dir=proj)
    PretrainTrainer(_model(), args, Stream()).train()
    losses = _losses(proj)
    assert len(losses) == 10 and all(l == l for l in losses) and losses[-1] < losses[0] - 0.2, losses


def test_resume_on_gpu_follows_the_uninterrupted_run(tmp_path):
    from rwkvtune_b200 import SFTConfig, SFTTrainer

    common = dict(ctx_len=64, micro_bsz=4, lr_init=3e-3, lr_final=1e-3, warmup_steps=0, accelerator="gpu", devices=1,
                  precision="bf16", grad_cp=0, epoch_save=1, save_total_limit=0)
    full = str(tmp_path / "full")
    SFTTrainer(_model(), SFTConfig(epoch_count=2, proj_dir=full, **common), _dataset()).train()
    resumed = str(tmp_path / "resumed")
    args = SFTConfig(epoch_count=2, proj_dir=resumed, resume_from_checkpoint=os.path.join(full, "rwkv7-epoch1"), **common)
    SFTTrainer(_model(), args, _dataset()).train()
    a, b = _losses(full), _losses(resumed)
    # fp32 master weights and moments come back exactly and the kernels sum in a fixed order
    assert len(b) == 8 and all(abs(x - y) < 2e-3 for x, y in zip(a[8:], b)), (a[8:], b)


_TWO_RANK_SFT = r'''
import os, sys, json, torch
sys.path.insert(0, os.environ["RWKV_ROOT"])
from rwkvtune_b200 import SFTConfig, SFTTrainer
from rwkvtune_b200.models import RWKVConfig, RWKV7Model
from rwkvtune_b200.parallel import shutdown

proj, strategy, resume = sys.argv[1], sys.argv[2], sys.argv[3]
torch.manual_seed(0)
model = RWKV7Model(RWKVConfig(n_layer=2, n_embd=256, vocab_size=512, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32))
with torch.no_grad():
    for n, p in model.named_parameters():
        if n.endswith(("output.weight", "ffn.value.weight")):
            p.normal_(0, 0.02)
g = torch.Generator().manual_seed(0)
base = torch.randint(1, 512, (4, 65), generator=g)
rows = []
for i in range(32):
    row = base[i % 4]
    rows.append({"input_ids": row[:-1].tolist(), "labels": row[1:].tolist()})
args = SFTConfig(ctx_len=64, micro_bsz=2, epoch_count=3, lr_init=3e-3, lr_final=1e-3, warmup_steps=2, accelerator="gpu",
                 devices=2, strategy=strategy, precision="bf16", proj_dir=proj, grad_cp=0, epoch_save=1,
                 resume_from_checkpoint=(resume if resume != "-" else None))
tr = SFTTrainer(model, args, rows)
tr.train()
tr.engine.check_health()
if tr.ctx.is_main:
    print(json.dumps({"world": tr.ctx.world_size, "transport": type(tr.engine.opt._p2p).__name__,
                      "samples_seen": tr.state["samples_seen"]}))
shutdown()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sft_trainer_on_two_gpus_saves_shards_and_resumes(tmp_path):
    """Two ranks through the public trainer: sharded optimiser over the fused peer-memory transport, one save point
    per epoch with one optimiser shard per rank, and a resumed run that continues the loss curve."""
    import subprocess
    import sys

    import socket

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def _free_port() -> int:
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]

    script = tmp_path / "sft2.py"
    script.write_text(_TWO_RANK_SFT)
    env = dict(os.environ, RWKV_ROOT=root, NCCL_NVLS_ENABLE="0")

    def run(proj, resume="-"):
        res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                              "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script), str(proj),
                              "deepspeed_stage_2", str(resume)], capture_output=True, text=True, env=env, timeout=300)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
        return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])

    full = tmp_path / "full"
    rec = run(full)
    assert rec["world"] == 2 and rec["transport"] != "NoneType", rec       # the fused transport, not the NCCL baseline
    losses = _losses(str(full))
    assert len(losses) == 24 and losses[-1] < losses[0] - 0.5, (losses[0], losses[-1])
    ck = full / "rwkv7-epoch2"
    assert sorted(os.listdir(ck / "trainer_state")) == ["meta.json", "rank0.pt", "rank1.pt"]
    resumed = tmp_path / "resumed"
    run(resumed, ck)
    tail = _losses(str(resumed))
    assert len(tail) == 8 and all(abs(x - y) < 5e-3 for x, y in zip(losses[16:], tail)), (losses[16:], tail)
