"""The bounds-recording build of the native library: an out-of-range data-dependent index is recorded (count, kernel
tag, index, limit) and skipped; nothing traps and the context stays usable; a clean training step records nothing."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CODE = r'''
import json, sys, torch
sys.path.insert(0, "%s")
from rwkvtune_b200 import ops
from rwkvtune_b200.ops import _ext
assert _ext.DEBUG_BUILD and _ext.lib_path().endswith("_debug.so")
out = {}
src = torch.arange(40, device="cuda", dtype=torch.float32).reshape(5, 8)
idx = torch.tensor([0, 4, 9, 2], device="cuda")          # 9 is outside the 5 rows
got = ops.gather_rows(src, idx)
torch.cuda.synchronize()
out["gather_rows"] = got.tolist()
out["events_after_bad_index"] = {k: list(v) for k, v in _ext.debug_events(reset=True).items()}
# a clean step through the whole model records nothing
from rwkvtune_b200.engine import EngineConfig, TrainEngine
from rwkvtune_b200.models import RWKVConfig, RWKV7Model
from rwkvtune_b200.parallel import DistContext
torch.manual_seed(0)
cfg = RWKVConfig(n_layer=2, n_embd=256, vocab_size=1024, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32)
eng = TrainEngine(RWKV7Model(cfg), EngineConfig(lr_init=1e-3, precision="bf16"), DistContext(device=torch.device("cuda", 0)))
ids = torch.randint(0, 1024, (2, 96), device="cuda")
labels = ids.roll(-1, 1).clone()
labels[:, :7] = -100
out["loss"] = float(eng.train_step(ids, labels, 1e-3))
out["events_after_clean_step"] = {k: list(v) for k, v in _ext.debug_events(reset=True).items()}
# a label outside the vocabulary is recorded by the loss-row kernel and contributes nothing
labels[0, 20] = 5000
out["loss_bad_label"] = float(eng.train_step(ids, labels, 1e-3))
out["events_after_bad_label"] = {k: list(v) for k, v in _ext.debug_events(reset=True).items()}
print(json.dumps(out))
''' % ROOT


def test_debug_build_records_out_of_range_indices_without_trapping():
    lib = os.path.join(ROOT, "rwkvtune_b200", "csrc", "librwkvtune_b200_debug.so")
    if not os.path.exists(lib):
        pytest.skip("debug library not built (python -m rwkvtune_b200.csrc.build --debug)")
    res = subprocess.run([sys.executable, "-c", _CODE], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, RWKVTUNE_DEBUG_LIB="1"))
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    rec = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert rec["gather_rows"][2] == [0.0] * 8 and rec["gather_rows"][1] == list(map(float, range(32, 40)))
    ev = rec["events_after_bad_index"]["gather"]
    assert ev[0] >= 1 and ev[1] == 1 and ev[2] == 9 and ev[3] == 5      # count, kernel tag, index, limit
    assert rec["events_after_clean_step"] == {}
    assert rec["loss"] == rec["loss"]
    bad = rec["events_after_bad_label"]["loss_rows"]
    assert bad[0] >= 1 and bad[1] == 11 and bad[2] == 5000 and bad[3] == 1024
    assert rec["loss_bad_label"] == rec["loss_bad_label"]                # finite: the row was simply not supervised
