"""Forward+backward replayed from a CUDA graph must train exactly like the eager path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(cuda_graph: bool, train_type: str, steps: int = 6):
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.parallel import DistContext

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    cfg = RWKVConfig(n_layer=2, n_embd=256, vocab_size=2048, dim_att_lora=32, dim_gate_lora=64, dim_mv_lora=32, ctx_len=512)
    model = RWKV7Model(cfg)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith(("output.weight", "ffn.value.weight", "w1", "a1", "v1", "g1")):
                p.normal_(0, 0.05)
    eng = TrainEngine(model, EngineConfig(lr_init=1e-3, precision="bf16", grad_cp=1, train_type=train_type, chunk_ctx=128,
                                          cuda_graph=cuda_graph), DistContext(device=dev))
    g = torch.Generator().manual_seed(1)
    T = 512 if train_type == "infctx" else 192
    losses = []
    for _ in range(steps):
        idx = torch.randint(0, 2048, (2, T), generator=g).to(dev)
        lab = torch.randint(0, 2048, (2, T), generator=g).to(dev)
        losses.append(float(eng.train_step(idx, lab, 1e-3)))
    return losses, len(eng._graphs)


@pytest.mark.parametrize("train_type", ["normal", "infctx"])
def test_graph_replay_trains_like_eager(train_type):
    eager, n0 = _run(False, train_type)
    graph, n1 = _run(True, train_type)
    assert n0 == 0 and n1 == 1            # one shape captured after the warm-up steps
    for a, b in zip(eager, graph):
        assert abs(a - b) <= 2e-3 * abs(a) + 1e-4, (eager, graph)


def test_run_wide_peak_survives_phase_resets():
    """Phases reset the allocator's peak counter for their own figure; the run-wide peak must still be the largest."""
    from rwkvtune_b200.engine.profiling import PhaseMonitor

    dev = torch.device("cuda", 0)
    mon = PhaseMonitor(dev)
    with mon.phase("big"):
        big = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
        del big
    with mon.phase("small"):
        small = torch.empty(1 << 20, dtype=torch.uint8, device=dev)
        del small
    assert mon.peak_gb["big"] > mon.peak_gb["small"]
    assert mon.peak_bytes() >= 64 << 20
    assert mon.peak_bytes() / 2**30 >= mon.peak_gb["big"] - 1e-6
