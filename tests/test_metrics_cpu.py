"""Metric sinks: the files every run writes, the external trackers (through a stand-in module), rank filtering."""
import json
import math
import os
import sys
import types

import pytest

from rwkvtune_b200.engine.metrics import MetricLogger


class _Tracker(types.ModuleType):
    """Stands in for ``swanlab`` / ``wandb``: records what the logger hands over."""

    def __init__(self, name):
        super().__init__(name)
        self.inits, self.logs, self.finished = [], [], 0

    def init(self, **kw):
        self.inits.append(kw)

    def log(self, scalars, step=None):
        self.logs.append((step, scalars))

    def finish(self):
        self.finished += 1


def test_files_written_by_every_run(tmp_path):
    proj = str(tmp_path / "run")
    log = MetricLogger(proj, config={"lr_init": 1e-3})
    rec = log.log_step(1, 2.5, 1e-3, tokens=4096, step_seconds=0.5)
    assert rec == {"loss": 2.5, "t_cost": 0.5, "kt_s": pytest.approx(8.192)}
    log.log_step(2, 2.0, 9e-4, tokens=2048, step_seconds=0.25, extra={"phase/forward_backward/seconds": 0.2})
    log.log_epoch(0, 2.25, 2)
    log.close()
    rows = [json.loads(l) for l in open(os.path.join(proj, "loss_data.jsonl"))]
    assert [set(r) for r in rows] == [{"loss", "t_cost", "kt_s"}] * 2 and rows[1]["loss"] == 2.0
    lines = open(os.path.join(proj, "train_log.txt")).read().splitlines()
    assert lines[0].startswith("NEW RUN ") and json.loads(lines[1]) == {"lr_init": 1e-3}
    epoch, mean, ppl, _stamp = lines[2].split()
    assert epoch == "0" and float(mean) == 2.25 and float(ppl) == pytest.approx(math.exp(2.25), rel=1e-4)
    # a second run in the same directory appends
    MetricLogger(proj).close()
    assert open(os.path.join(proj, "train_log.txt")).read().count("NEW RUN") == 2


@pytest.mark.parametrize("name", ["swanlab", "wandb"])
def test_external_tracker_receives_named_scalars(tmp_path, monkeypatch, name):
    fake = _Tracker(name)
    monkeypatch.setitem(sys.modules, name, fake)
    proj = str(tmp_path / "proj-x")
    log = MetricLogger(proj, report_to=name, run_name="trial", config={"a": 1})
    assert fake.inits == [{"project": "proj-x", "name": "trial", "config": {"a": 1}}]
    log.log_step(3, 1.5, 2e-4, tokens=1000, step_seconds=1.0, extra={"clip_ratio": 0.1})
    log.log_epoch(1, 1.5, 3)
    log.log_scalars({"train/reward/mean": 0.3}, 3)
    log.close()
    step, scalars = fake.logs[0]
    assert step == 3 and scalars["train/loss"] == 1.5 and scalars["train/lr"] == 2e-4
    assert scalars["train/throughput_kt_s"] == pytest.approx(1.0) and scalars["clip_ratio"] == 0.1
    assert fake.logs[1][1]["train/epoch_perplexity"] == pytest.approx(math.exp(1.5))
    assert fake.logs[2] == (3, {"train/reward/mean": 0.3}) and fake.finished == 1


def test_missing_tracker_is_reported_not_fatal(tmp_path, monkeypatch, capsys):
    monkeypatch.setitem(sys.modules, "swanlab", None)          # import raises ImportError
    log = MetricLogger(str(tmp_path / "p"), report_to="swanlab")
    assert log.ext is None and "swanlab unavailable" in capsys.readouterr().out
    assert log.log_step(1, 1.0, 1e-3, 10, 1.0)["loss"] == 1.0


def test_other_ranks_write_nothing(tmp_path):
    proj = str(tmp_path / "quiet")
    log = MetricLogger(proj, report_to="tensorboard", is_main=False)
    rec = log.log_step(1, 3.0, 1e-3, tokens=100, step_seconds=0.1)
    log.log_epoch(0, 3.0, 1)
    log.log_scalars({"x": 1.0}, 1)
    log.close()
    assert rec["loss"] == 3.0 and not os.path.exists(proj)


def test_perplexity_is_capped_for_diverged_losses(tmp_path):
    proj = str(tmp_path / "big")
    log = MetricLogger(proj)
    log.log_epoch(0, 1e6, 1)
    assert float(open(os.path.join(proj, "train_log.txt")).read().splitlines()[-1].split()[2]) == pytest.approx(math.exp(50.0))
