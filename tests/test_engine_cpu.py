"""Engine-level behaviour on CPU: infinite-context steps with masked chunks, phase timers, bucket planning, the N-step
profiler, checkpoint publication / rotation / lookup."""
import pytest
import torch

from rwkvtune_b200.engine import EngineConfig, TrainEngine
from rwkvtune_b200.models import RWKVConfig, RWKV7Model
from rwkvtune_b200.parallel import DistContext


def _engine(**kw):
    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=64, vocab_size=128, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16)
    return TrainEngine(RWKV7Model(cfg), EngineConfig(lr_init=1e-3, precision="fp32", train_type="infctx", chunk_ctx=16,
                                                     **kw), DistContext())


def _batch():
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(1, 128, (2, 48), generator=g)
    labels = idx.roll(-1, 1).clone()
    labels[:, :16] = -100            # the whole first chunk is prompt
    return idx, labels


def test_full_bptt_skips_fully_masked_chunks_and_divides_by_all_chunks():
    idx, labels = _batch()
    eng = _engine(truncated_bptt=False)
    loss = eng.train_step(idx, labels, 1e-3)
    assert torch.isfinite(loss)
    # the same number from the plain statements: two supervised chunks, each a mean over its own tokens, over 3 chunks
    ref = _engine(truncated_bptt=False)
    m = ref.model
    with torch.no_grad():
        logits = m(idx)
    per_chunk = []
    for c in (1, 2):
        sl = slice(16 * c, 16 * (c + 1))
        per_chunk.append(torch.nn.functional.cross_entropy(logits[:, sl].reshape(-1, 128), labels[:, sl].reshape(-1)))
    assert abs(float(loss) - float(sum(per_chunk) / 3)) < 1e-4
    truncated = _engine(truncated_bptt=True).train_step(idx, labels, 1e-3)
    assert abs(float(truncated) - float(loss)) < 1e-4


def test_nothing_supervised_is_a_zero_loss_step_not_a_nan():
    idx, labels = _batch()
    labels[:] = -100
    for truncated in (True, False):
        loss = _engine(truncated_bptt=truncated).train_step(idx, labels, 1e-3)
        assert float(loss) == 0.0


def test_phase_monitor_collects_engine_phases():
    idx, labels = _batch()
    eng = _engine()
    eng.train_step(idx, labels, 1e-3)
    sc = eng.phases.scalars()
    assert sc["phase/forward_backward/seconds"] > 0 and "phase/reduce_optimizer/seconds" in sc
    assert eng.phases.scalars() == {}          # reset after reading


def test_bucket_plan_covers_the_space_with_whole_parameters():
    from rwkvtune_b200.parallel.p2p import plan_buckets

    segs, off = [], 0
    for n in (100, 4000, 128, 9000, 256, 256, 12000, 64):
        segs.append((off, n))
        off += (n + 127) // 128 * 128
    padded = (off + 1023) // 1024 * 1024
    bounds, seg_bucket = plan_buckets(segs, padded, 8000)
    assert bounds[0] == 0 and bounds[-1] == padded and bounds == sorted(bounds)
    assert len(seg_bucket) == len(segs) and seg_bucket == sorted(seg_bucket)
    starts = {s for s, _ in segs} | {padded}
    assert all(b in starts for b in bounds)                      # buckets start at parameter boundaries
    for (start, n), b in zip(segs, seg_bucket):
        assert bounds[b] <= start and start + n <= bounds[b + 1]
    assert len(bounds) - 1 >= 3
    one, sb = plan_buckets(segs, padded, 10**9)
    assert one == [0, padded] and set(sb) == {0}
    many, _ = plan_buckets(segs, padded, 1, max_buckets=4)       # capped
    assert len(many) - 1 <= 4


def test_step_profiler_writes_a_table_for_the_requested_steps(tmp_path, monkeypatch):
    import os

    from rwkvtune_b200.engine.profiling import StepProfiler, profile_steps_requested

    class Args:
        profile_steps = 2

    monkeypatch.delenv("RWKVTUNE_PROFILE", raising=False)
    assert profile_steps_requested(Args()) == 2 and profile_steps_requested(object()) == 0
    monkeypatch.setenv("RWKVTUNE_PROFILE", "5")
    assert profile_steps_requested(Args()) == 5                     # the environment wins
    monkeypatch.setenv("RWKVTUNE_PROFILE", "off")
    assert profile_steps_requested(Args()) == 2

    prof = StepProfiler(2, str(tmp_path / "run"), skip=1)
    a = torch.randn(64, 64)
    for step in range(5):
        prof.step_begin()
        (a @ a).sum()
        prof.step_end()
        # recording spans exactly steps 1 and 2
        assert (prof.prof is not None) == (step == 1)
    text = open(os.path.join(str(tmp_path / "run"), "profile_kernels.txt")).read()
    assert text.startswith("2 training steps after 1 warm-up steps") and "aten::mm" in text
    quiet = StepProfiler(1, str(tmp_path / "other"), skip=0, is_main=False)
    quiet.step_begin()
    quiet.step_end()
    assert not os.path.exists(str(tmp_path / "other"))
    off = StepProfiler(0, str(tmp_path / "off"))
    off.step_begin()
    off.step_end()
    assert off.prof is None and not os.path.exists(str(tmp_path / "off"))


def test_trainer_profile_steps_switch(tmp_path, monkeypatch):
    import os

    from rwkvtune_b200 import SFTConfig, SFTTrainer
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model

    monkeypatch.delenv("RWKVTUNE_PROFILE", raising=False)
    torch.manual_seed(0)
    model = RWKV7Model(RWKVConfig(n_layer=1, n_embd=64, vocab_size=64, dim_att_lora=8, dim_gate_lora=8, dim_mv_lora=8))
    rows = [{"input_ids": list(range(1, 17)), "labels": list(range(2, 18))} for _ in range(12)]
    proj = str(tmp_path / "p")
    args = SFTConfig(ctx_len=16, micro_bsz=2, epoch_count=1, accelerator="cpu", precision="fp32", proj_dir=proj, grad_cp=0,
                     profile_steps=1)
    SFTTrainer(model, args, rows).train()
    text = open(os.path.join(proj, "profile_kernels.txt")).read()
    assert text.startswith("1 training steps after 3 warm-up steps") and "aten::" in text


def test_checkpoint_publication_replacement_rotation_and_lookup(tmp_path):
    import os
    import time

    from rwkvtune_b200.engine import checkpoint as ckpt
    from rwkvtune_b200.parallel import DistContext

    ctx = DistContext()
    final = str(tmp_path / "rwkv7-batch1")

    def writer(text):
        def write(tmp):
            with open(os.path.join(tmp, "model.pth"), "w") as fh:
                fh.write(text)
        return write

    ckpt.atomic_checkpoint(final, ctx, writer("first"))
    ckpt.atomic_checkpoint(final, ctx, writer("second"))                       # same name again: replaced, nothing left over
    assert open(os.path.join(final, "model.pth")).read() == "second"
    assert sorted(os.listdir(tmp_path)) == ["rwkv7-batch1"]

    def failing(tmp):
        raise OSError("disk full")

    with pytest.raises(OSError, match="disk full"):
        ckpt.atomic_checkpoint(final, ctx, failing)
    assert open(os.path.join(final, "model.pth")).read() == "second" and sorted(os.listdir(tmp_path)) == ["rwkv7-batch1"]

    for i in (2, 3, 4):
        d = tmp_path / f"rwkv7-batch{i}"
        (d / ckpt.STATE_DIR).mkdir(parents=True)
        now = time.time() + i
        os.utime(d, (now, now))
    (tmp_path / "rwkv7-batch9.tmp").mkdir()                                    # an unfinished save is not a candidate
    assert ckpt.rotate_checkpoints(str(tmp_path), 0) == []
    removed = ckpt.rotate_checkpoints(str(tmp_path), 2)
    assert sorted(os.path.basename(r) for r in removed) == ["rwkv7-batch1", "rwkv7-batch2"]
    assert ckpt.find_checkpoint(str(tmp_path)).endswith("rwkv7-batch4")        # a parent directory: the newest child
    assert ckpt.find_checkpoint(str(tmp_path / "rwkv7-batch3")).endswith("rwkv7-batch3")
    weights = tmp_path / "plain.pth"
    weights.write_text("x")
    assert ckpt.find_checkpoint(str(weights)) == str(weights)                  # a bare file is taken as it is
    assert ckpt.find_checkpoint(str(tmp_path / "nowhere")) is None and ckpt.find_checkpoint(None) is None
    assert ckpt.read_meta(str(tmp_path / "rwkv7-batch3")) == {}
