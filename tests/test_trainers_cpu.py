"""SFT/Pretrain trainers end to end on CPU: loss goes down, checkpoint layout, resume (exact, "latest", from adapter or
full-weight files), LoRA, CLI round trip, argument validation, the checkpoint-tuning decision."""
import json
import os

import pytest
import torch

from rwkvtune_b200 import AutoModel, LoraConfig, PretrainConfig, PretrainTrainer, SFTConfig, SFTTrainer
from rwkvtune_b200.models import RWKVConfig, RWKV7Model


def _dataset(n=24, T=32, V=128, seed=0):
    g = torch.Generator().manual_seed(seed)
    base = torch.randint(1, V, (4, T + 1), generator=g)
    out = []
    for i in range(n):
        row = base[i % 4]
        labels = row[1:].clone()
        labels[:4] = -100
        out.append({"input_ids": row[:-1].tolist(), "labels": labels.tolist()})
    return out


def _model():
    torch.manual_seed(0)
    return RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16))


def _losses(proj):
    return [json.loads(l)["loss"] for l in open(os.path.join(proj, "loss_data.jsonl"))]


def test_sft_trainer_trains_and_saves(tmp_path):
    proj = str(tmp_path / "sft")
    args = SFTConfig(ctx_len=32, micro_bsz=4, epoch_count=3, lr_init=5e-3, lr_final=1e-3, warmup_steps=2,
                     accelerator="cpu", precision="fp32", proj_dir=proj, grad_cp=0, save_total_limit=2)
    tr = SFTTrainer(_model(), args, _dataset())
    tr.train()
    losses = _losses(proj)
    assert len(losses) == 18 and losses[-1] < losses[0] - 0.5
    kept = sorted(d for d in os.listdir(proj) if d.startswith("rwkv7-"))
    assert kept == ["rwkv7-epoch2", "rwkv7-epoch3"]
    ck = os.path.join(proj, "rwkv7-epoch3")
    assert {"config.json", "model.pth", "trainer_state"} <= set(os.listdir(ck))
    meta = json.load(open(os.path.join(ck, "trainer_state", "meta.json")))
    assert meta["samples_seen"] == 72 and meta["devices"] == 1 and meta["micro_bsz"] == 4
    reloaded = AutoModel.from_pretrained(ck)
    idx = torch.tensor([_dataset()[0]["input_ids"]])
    assert torch.allclose(reloaded(idx), tr.model(idx), atol=1e-5)
    assert tr.save_model().endswith("final") and os.path.exists(os.path.join(proj, "final", "model.pth"))


def test_resume_reproduces_uninterrupted_run(tmp_path):
    common = dict(ctx_len=32, micro_bsz=4, lr_init=3e-3, lr_final=1e-3, warmup_steps=0, accelerator="cpu",
                  precision="fp32", grad_cp=0, epoch_save=1, save_total_limit=0)
    full = str(tmp_path / "full")
    SFTTrainer(_model(), SFTConfig(epoch_count=2, proj_dir=full, **common), _dataset()).train()
    part = str(tmp_path / "part")
    SFTTrainer(_model(), SFTConfig(epoch_count=2, proj_dir=part, **common), _dataset()).train()
    # drop the second epoch's records, resume from the epoch-1 checkpoint in a fresh trainer
    resumed = str(tmp_path / "resumed")
    args = SFTConfig(epoch_count=2, proj_dir=resumed, resume_from_checkpoint=os.path.join(part, "rwkv7-epoch1"), **common)
    SFTTrainer(_model(), args, _dataset()).train()
    a, b = _losses(full), _losses(resumed)
    assert len(b) == 6 and all(abs(x - y) < 1e-4 for x, y in zip(a[6:], b))


def test_lora_sft_saves_adapter_and_merges(tmp_path):
    from rwkvtune_b200.cli import merge_lora
    from rwkvtune_b200.utils import create_model_hub

    base = _model()
    with torch.no_grad():
        for n, p in base.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight")):
                p.normal_(0, 0.05)
    raw = str(tmp_path / "raw.pth")
    torch.save(base.state_dict(), raw)
    hub = create_model_hub(str(tmp_path / "hub"), model_file=raw)
    assert json.load(open(os.path.join(hub, "config.json")))["n_embd"] == 64
    proj = str(tmp_path / "lora")
    args = SFTConfig(ctx_len=32, micro_bsz=4, epoch_count=2, lr_init=5e-3, warmup_steps=0, accelerator="cpu",
                     precision="fp32", proj_dir=proj, grad_cp=0)
    tr = SFTTrainer(hub, args, _dataset(), lora_config=LoraConfig(r=4, lora_alpha=8))
    tr.train()
    ck = os.path.join(proj, "rwkv7-epoch2")
    assert {"adapter_model.bin", "adapter_config.json", "lora_config.json"} <= set(os.listdir(ck))
    keys = torch.load(os.path.join(ck, "adapter_model.bin")).keys()
    assert any("lora_A" in k for k in keys) and any("ln1" in k for k in keys)
    out = str(tmp_path / "merged")
    assert merge_lora.main(["-b", hub, "-l", ck, "-o", out, "--precision", "fp32"]) == 0
    merged = AutoModel.from_pretrained(out)
    idx = torch.tensor([_dataset()[0]["input_ids"]])
    assert torch.allclose(merged(idx), tr.model(idx), atol=1e-4)


def test_pretrain_trainer_infctx_iterable(tmp_path):
    class Stream:
        def __iter__(self):
            return iter(_dataset(16))

    proj = str(tmp_path / "pre")
    args = PretrainConfig(ctx_len=32, micro_bsz=2, epoch_count=1, epoch_steps=6, train_type="infctx", chunk_ctx=16,
                          lr_init=5e-3, warmup_steps=0, accelerator="cpu", precision="fp32", proj_dir=proj)
    PretrainTrainer(_model(), args, Stream()).train()
    losses = _losses(proj)
    assert len(losses) == 6 and losses[-1] < losses[0]


class _FakePanels:
    """Stands in for a ZeRO-3 sharded weight: the module holds an empty tensor, the full matrix comes from here."""

    def __init__(self, full):
        self.full = full.clone()
        self.calls = 0

    def full_weight(self):
        self.calls += 1
        return self.full


def test_full_and_merged_saves_reassemble_sharded_weights(tmp_path):
    from rwkvtune_b200.peft import get_peft_model
    from rwkvtune_b200.training.model_save_utils import save_model_or_adapter

    model = get_peft_model(_model(), LoraConfig(r=4, lora_alpha=8))
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)
    expected = model.get_merged_state_dict()
    idx = torch.tensor([_dataset()[0]["input_ids"]])
    want = model(idx)
    # shard: every adapted projection loses its base weight, as Zero3ShardedLinears does on a multi-GPU stage-3 run
    fakes = []
    for name, m in model.named_modules():
        if hasattr(m, "base_layer"):
            m._sharded = _FakePanels(m.base_layer.weight.data)
            m.base_layer.weight.data = torch.empty(0)
            fakes.append(m._sharded)
    assert fakes and all(f.calls == 0 for f in fakes)
    got = model.get_merged_state_dict()
    assert set(got) == set(expected)
    for k in expected:
        assert got[k].shape == expected[k].shape and torch.allclose(got[k], expected[k], atol=1e-6), k
    assert all(m.base_layer.weight.numel() == 0 for _, m in model.named_modules() if hasattr(m, "base_layer"))
    out = str(tmp_path / "both")
    save_model_or_adapter(model, out, None, "both")
    assert os.path.exists(os.path.join(out, "adapter_model.bin"))
    merged = AutoModel.from_pretrained(os.path.join(out, "merged"))
    assert torch.allclose(merged(idx), want, atol=1e-4)
    full = str(tmp_path / "full")
    save_model_or_adapter(model, full, None, "full")
    assert torch.allclose(AutoModel.from_pretrained(full)(idx), want, atol=1e-4)


def test_truncated_optimizer_shard_falls_back_to_weights_only_resume(tmp_path, capsys):
    common = dict(ctx_len=32, micro_bsz=4, lr_init=3e-3, lr_final=1e-3, warmup_steps=0, accelerator="cpu",
                  precision="fp32", grad_cp=0, epoch_save=1, save_total_limit=0)
    first = str(tmp_path / "first")
    SFTTrainer(_model(), SFTConfig(epoch_count=1, proj_dir=first, **common), _dataset()).train()
    ck = os.path.join(first, "rwkv7-epoch1")
    shard = os.path.join(ck, "trainer_state", "rank0.pt")
    raw = open(shard, "rb").read()
    open(shard, "wb").write(raw[:len(raw) // 3])          # the file was cut short
    resumed = str(tmp_path / "resumed")
    args = SFTConfig(epoch_count=2, proj_dir=resumed, resume_from_checkpoint=ck, **common)
    SFTTrainer(_model(), args, _dataset()).train()
    out = capsys.readouterr().out
    assert "unreadable" in out and "weights only" in out
    losses = _losses(resumed)
    assert len(losses) == 6 and all(l == l for l in losses)      # the second epoch ran from the saved weights
    # a missing meta file means "no trainer state": also a clean weights-only resume
    os.remove(os.path.join(ck, "trainer_state", "meta.json"))
    again = str(tmp_path / "again")
    SFTTrainer(_model(), SFTConfig(epoch_count=1, proj_dir=again, resume_from_checkpoint=ck, **common), _dataset()).train()
    assert len(_losses(again)) == 6


def test_resume_latest_picks_the_newest_save_point_under_proj_dir(tmp_path, capsys):
    proj = str(tmp_path / "run")
    common = dict(ctx_len=32, micro_bsz=4, lr_init=3e-3, warmup_steps=0, accelerator="cpu", precision="fp32", grad_cp=0,
                  epoch_save=1, save_total_limit=0, proj_dir=proj)
    PretrainTrainer(_model(), PretrainConfig(epoch_count=2, **common), _dataset()).train()
    assert {"rwkv7-epoch1", "rwkv7-epoch2"} <= set(os.listdir(proj))
    capsys.readouterr()
    tr = PretrainTrainer(_model(), PretrainConfig(epoch_count=3, resume_from_checkpoint="latest", **common), _dataset())
    tr.train()
    out = capsys.readouterr().out
    assert "rwkv7-epoch2" in out and "with optimizer state" in out and "samples_seen=48" in out
    assert tr.state["samples_seen"] == 72 and len(_losses(proj)) == 18          # 12 records of the first run + 6 new
    # a parent directory resolves the same way; a path without any save point is an error, not a fresh start
    from rwkvtune_b200.engine import checkpoint as ckpt
    assert ckpt.find_checkpoint(proj).endswith("rwkv7-epoch3")
    with pytest.raises(FileNotFoundError):
        PretrainTrainer(_model(), PretrainConfig(epoch_count=1, resume_from_checkpoint=str(tmp_path / "nowhere"),
                                                 **{**common, "proj_dir": str(tmp_path / "other")}), _dataset()).train()


def test_checkpoint_tuning_is_asked_for_only_when_it_is_safe(monkeypatch, capsys):
    """The trainers hand the choice of recomputed blocks to the engine after the first step - on a GPU, in normal mode,
    with ``grad_cp=1``, and only if every rank's first batch had the full length."""
    import types

    calls = []

    def trainer(agree=True, device="cuda", **cfg):
        args = SFTConfig(ctx_len=64, micro_bsz=4, accelerator="cpu", precision="fp32", **cfg)
        tr = SFTTrainer(_model(), args, _dataset())
        tr.ctx = types.SimpleNamespace(device=types.SimpleNamespace(type=device), is_main=True,
                                       all_agree=lambda ok: bool(ok) and agree)
        tr.engine = types.SimpleNamespace(model=types.SimpleNamespace(config=types.SimpleNamespace(n_layer=2)),
                                          autotune_checkpointing=lambda b, t: calls.append((b, t)) or 1)
        return tr

    monkeypatch.delenv("RWKVTUNE_GRAD_CP_AUTO", raising=False)
    trainer(grad_cp=1)._tune_checkpointing(64)
    assert calls == [(4, 64)] and "1 of 2 blocks recomputed" in capsys.readouterr().out
    trainer(grad_cp=0)._tune_checkpointing(64)
    trainer(grad_cp=1, train_type="infctx", chunk_ctx=32)._tune_checkpointing(64)
    trainer(grad_cp=1, device="cpu")._tune_checkpointing(64)
    trainer(grad_cp=1)._tune_checkpointing(48)                  # a short first batch says nothing about the longest one
    trainer(grad_cp=1, agree=False)._tune_checkpointing(64)     # another rank's first batch was short
    monkeypatch.setenv("RWKVTUNE_GRAD_CP_AUTO", "0")
    trainer(grad_cp=1)._tune_checkpointing(64)
    assert calls == [(4, 64)]


def test_dataset_and_mode_validation_errors(tmp_path):
    cfg = dict(ctx_len=32, micro_bsz=4, accelerator="cpu", precision="fp32", proj_dir=str(tmp_path / "v"))
    with pytest.raises(ValueError, match="train_dataset is required"):
        SFTTrainer(_model(), SFTConfig(**cfg), None)
    with pytest.raises(ValueError, match="empty"):
        SFTTrainer(_model(), SFTConfig(**cfg), [])
    with pytest.raises(TypeError, match="map-style"):
        SFTTrainer(_model(), SFTConfig(**cfg), iter(_dataset()))

    class Columns(list):
        column_names = ["input_ids", "text"]

    with pytest.raises(ValueError, match="lacks columns"):
        SFTTrainer(_model(), SFTConfig(**cfg), Columns(_dataset()))

    class Stream:
        def __iter__(self):
            return iter(_dataset())

    with pytest.raises(ValueError, match="epoch_steps"):
        PretrainTrainer(_model(), PretrainConfig(**cfg), Stream()).train()
    with pytest.raises(ValueError, match="too small"):
        SFTTrainer(_model(), SFTConfig(**cfg), _dataset(3)).train()
    with pytest.raises(ValueError, match="accumulate_grad_batches"):
        PretrainTrainer(_model(), PretrainConfig(train_type="infctx", chunk_ctx=16, accumulate_grad_batches=2, **cfg),
                        _dataset()).train()


def test_adapter_runs_save_per_batch_and_resume_from_directory_file_or_full_weights(tmp_path, capsys):
    common = dict(ctx_len=32, micro_bsz=4, lr_init=5e-3, warmup_steps=0, accelerator="cpu", precision="fp32", grad_cp=0,
                  save_total_limit=0)
    first = str(tmp_path / "first")
    tr = SFTTrainer(_model(), SFTConfig(epoch_count=1, proj_dir=first, save_every_n_batches=2, **common), _dataset(),
                    lora_config=LoraConfig(r=4, lora_alpha=8))
    tr.train()
    assert {"rwkv7-batch2", "rwkv7-batch4", "rwkv7-batch6", "rwkv7-epoch1"} <= set(os.listdir(first))
    ck = os.path.join(first, "rwkv7-epoch1")
    idx = torch.tensor([_dataset()[0]["input_ids"]])
    want = tr.model(idx)

    def resumed(source, epochs=1):
        t = SFTTrainer(_model(), SFTConfig(epoch_count=epochs, proj_dir=str(tmp_path / f"r{abs(hash(source)) % 9999}"),
                                           resume_from_checkpoint=source, **common), _dataset(),
                       lora_config=LoraConfig(r=4, lora_alpha=8))
        t.train()
        return t

    a = resumed(ck)                                                     # the checkpoint directory (adapter inside)
    assert a.state["samples_seen"] == 24 and torch.allclose(a.model(idx), want, atol=1e-5)
    capsys.readouterr()
    b = resumed(os.path.join(ck, "adapter_model.bin"))                  # the bare adapter file: weights only, a fresh epoch
    out = capsys.readouterr().out
    assert "adapter_model.bin (weights only); samples_seen=0" in out and "step 6/6" in out
    assert not torch.allclose(b.model(idx), want, atol=1e-5)            # it trained on from the loaded adapter
    full = str(tmp_path / "plain.pth")                                  # a plain full-weight file into an adapter model
    torch.save(_model().state_dict(), full)
    c = SFTTrainer(_model(), SFTConfig(epoch_count=1, proj_dir=str(tmp_path / "c"), resume_from_checkpoint=full, **common),
                   _dataset(), lora_config=LoraConfig(r=4, lora_alpha=8))
    c.train()
    assert any("lora_A" in n for n, _ in c.model.named_parameters())
    empty = tmp_path / "emptyck"
    (empty / "trainer_state").mkdir(parents=True)
    with pytest.raises(FileNotFoundError, match="neither model weights nor adapter"):
        SFTTrainer(_model(), SFTConfig(epoch_count=1, proj_dir=str(tmp_path / "d"), resume_from_checkpoint=str(empty), **common),
                   _dataset()).train()
