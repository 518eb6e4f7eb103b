"""User callbacks of the trainers: hook order, arguments, and Lightning-style signatures; the phase helper."""
import torch

from rwkvtune_b200 import LoraConfig, SFTConfig, SFTTrainer
from rwkvtune_b200.models import RWKVConfig, RWKV7Model
from rwkvtune_b200.training.callbacks import CallbackList, TrainingCallback
from rwkvtune_b200.training.grpo import get_gpu_memory_info, monitor_memory_and_time


def _model(**kw):
    torch.manual_seed(0)
    return RWKV7Model(RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16, **kw))


def _dataset(n=8, T=16, V=128):
    g = torch.Generator().manual_seed(0)
    rows = torch.randint(1, V, (n, T + 1), generator=g)
    return [{"input_ids": r[:-1].tolist(), "labels": r[1:].tolist()} for r in rows]


class _Recorder(TrainingCallback):
    def __init__(self):
        self.events = []

    def on_train_start(self, trainer):
        self.events.append(("start", trainer.engine is not None))

    def on_train_batch_start(self, trainer, batch, batch_idx):
        ids = batch["input_ids"]      # a tensor in the supervised trainers, the prompts' token lists in GRPO
        self.events.append(("batch_start", batch_idx, tuple(ids.shape) if hasattr(ids, "shape") else len(ids)))

    def on_train_batch_end(self, trainer, outputs, batch, batch_idx):
        self.events.append(("batch_end", batch_idx, outputs["loss"] == outputs["loss"], outputs["lr"] > 0))

    def on_train_epoch_end(self, trainer, epoch):
        self.events.append(("epoch_end", epoch))

    def on_save_checkpoint(self, trainer, path):
        self.events.append(("save", path.rsplit("/", 1)[-1]))

    def on_train_end(self, trainer):
        self.events.append(("end",))


class _LightningStyle:
    """Written against ``hook(trainer, pl_module, ...)``; no base class."""

    def __init__(self):
        self.seen = []

    def on_train_batch_end(self, trainer, pl_module, outputs, batch, batch_idx):
        self.seen.append((sum(p.numel() for p in pl_module.parameters()) > 0, batch_idx, float(outputs["loss"])))


def test_sft_trainer_calls_hooks_in_order(tmp_path):
    rec, lit = _Recorder(), _LightningStyle()
    args = SFTConfig(ctx_len=16, micro_bsz=4, epoch_count=2, lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="cpu",
                     precision="fp32", proj_dir=str(tmp_path / "p"), grad_cp=0, epoch_save=1)
    SFTTrainer(_model(), args, _dataset(), callbacks=[rec, lit]).train()
    kinds = [e[0] for e in rec.events]
    assert kinds == ["start", "batch_start", "batch_end", "batch_start", "batch_end", "epoch_end", "save",
                     "batch_start", "batch_end", "batch_start", "batch_end", "epoch_end", "save", "end"]
    assert rec.events[0] == ("start", True)
    assert rec.events[1] == ("batch_start", 0, (4, 16)) and rec.events[2] == ("batch_end", 0, True, True)
    assert [e[1] for e in rec.events if e[0] == "save"] == ["rwkv7-epoch1", "rwkv7-epoch2"]
    assert [s[1] for s in lit.seen] == [0, 1, 0, 1] and all(s[0] for s in lit.seen)


def test_grpo_trainer_calls_hooks(tmp_path):
    from rwkvtune_b200 import GRPOConfig, GRPOTrainer

    class Tok:
        eos_token_id = 7
        pad_token_id = 0

        def encode(self, s):
            return [ord(c) % 100 + 8 for c in s]

        def decode(self, ids):
            return " ".join(str(int(i)) for i in ids)

    model = _model(eos_token_id=7)
    data = [{"prompt": f"p{i}", "input_ids": [10 + i, 11 + i, 12 + i]} for i in range(2)]
    args = GRPOConfig(micro_bsz=2, num_generations=2, steps_per_generation=1, max_prompt_length=8, max_completion_length=4,
                      beta=0.0, lr_init=1e-3, lr_final=1e-4, warmup_steps=0, accelerator="cpu", precision="fp32",
                      proj_dir=str(tmp_path / "g"), epoch_count=1, log_steps=1)
    rec = _Recorder()
    steps = []

    class OnlyStepEnd:
        def on_step_end(self, trainer, metrics):
            steps.append(metrics["train_loss"])

    GRPOTrainer(model, lambda prompts, completions, **k: [float(len(c)) for c in completions], args, data,
                processing_class=Tok(), peft_config=LoraConfig(r=4, lora_alpha=8), callbacks=[rec, OnlyStepEnd()]).train()
    kinds = [e[0] for e in rec.events]
    assert kinds[0] == "start" and kinds[-1] == "end" and kinds[-2] == "save"
    assert kinds.count("batch_start") == kinds.count("batch_end") == len(steps) >= 1
    assert "epoch_end" in kinds


def test_callback_list_skips_missing_hooks_and_keeps_order():
    calls = []

    class A:
        def on_train_start(self, trainer):
            calls.append("a")

    class B:
        pass

    class C:
        def on_train_start(self, trainer, pl_module):
            calls.append(("c", pl_module))

    class T:
        model = "the-model"

    cl = CallbackList([A(), B()])
    cl.append(C())
    cl.fire("on_train_start", T())
    cl.fire("on_train_end", T())
    assert calls == ["a", ("c", "the-model")] and len(cl) == 3


def test_phase_helper_prints_one_line_on_cpu():
    lines = []
    with monitor_memory_and_time(3, "rewards", sink=lines.append) as mon:
        sum(range(1000))
    assert len(lines) == 1 and lines[0].startswith("[Rank 3] rewards: ") and lines[0].endswith(" s")
    assert mon.calls["rewards"] == 1
    if not torch.cuda.is_available():
        assert get_gpu_memory_info() is None
