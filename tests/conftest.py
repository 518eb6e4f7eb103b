"""Shared fixtures.  GPU-only tests carry ``@pytest.mark.gpu``; everything else runs on CPU."""
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: longer-running CPU test")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _reference_dir():
    cand = os.environ.get("RWKVTUNE_REFERENCE_DIR", os.path.join(ROOT, "baseline", "_ref"))
    return cand if os.path.isdir(os.path.join(cand, "rwkvtune")) else None


@pytest.fixture(scope="session")
def reference_pkg():
    """The unmodified reference package, importable with a stub in place of ``lightning``
    (which is not installed).  Only its model, operators and pure functions are used as oracles."""
    ref = _reference_dir()
    if ref is None:
        pytest.skip("reference package not installed under baseline/_ref")
    os.environ.setdefault("RWKV_DEVICE", "cpu")
    if ref not in sys.path:
        sys.path.insert(0, ref)
    for name in ("lightning", "lightning.pytorch", "lightning.pytorch.callbacks", "lightning.pytorch.strategies",
                 "lightning.pytorch.loggers", "lightning.pytorch.utilities"):
        if name not in sys.modules:
            mod = types.ModuleType(name)
            mod.__path__ = []
            sys.modules[name] = mod
    L = sys.modules["lightning"]
    class _Stub:  # minimal base classes referenced at import time
        def __init__(self, *a, **k):
            pass
    for attr in ("LightningModule", "Trainer", "Callback", "LightningDataModule"):
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
    try:
        import rwkvtune.models.rwkv7.model as ref_model  # noqa: F401
    except Exception as exc:  # pragma: no cover - depends on the local install
        pytest.skip(f"reference import failed: {exc}")
    import rwkvtune
    return rwkvtune
