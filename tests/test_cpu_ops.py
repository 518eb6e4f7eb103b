"""The host-CPU fast paths against the plain statements they replace."""
import pytest
import torch

from rwkvtune_b200 import ops
from rwkvtune_b200.ops import cpu_ops, reference


def _inputs(B, T, H, N, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    C = H * N
    r, k, v = torch.randn(B, T, C, generator=g), torch.randn(B, T, C, generator=g) * 0.3, torch.randn(B, T, C, generator=g)
    w = -0.5 - torch.rand(B, T, C, generator=g)
    kk = torch.nn.functional.normalize(torch.randn(B, T, H, N, generator=g), dim=-1).reshape(B, T, C)
    a, b = -kk, kk * torch.rand(B, T, C, generator=g)
    state = torch.randn(B, H, N, N, generator=g) * 0.2
    return [t.to(dtype) for t in (r, w, k, v, a, b)], state


@pytest.fixture(params=["native", "torch"])
def form(request, monkeypatch):
    """Both forms of the fast recurrence: inside the native library, and the pure-PyTorch one it falls back to."""
    if request.param == "torch":
        monkeypatch.setattr(cpu_ops, "_NATIVE", None)
        monkeypatch.setattr(cpu_ops, "_NATIVE_TRIED", True)
    elif cpu_ops._native_lib() is None:
        pytest.skip("native library not built")
    return request.param


@pytest.mark.parametrize("shape,with_state", [((2, 9, 2, 8), True), ((1, 17, 3, 16), False), ((2, 33, 2, 64), True),
                                              ((1, 1, 1, 64), True), ((1, 16, 1, 8), True), ((2, 48, 1, 8), False)])
def test_recurrence_node_matches_the_traced_statement(form, shape, with_state):
    B, T, H, N = shape
    ins, s0 = _inputs(B, T, H, N)
    s0 = s0 if with_state else None
    g = torch.Generator().manual_seed(5)
    dy, ds = torch.randn(B, T, H * N, generator=g), torch.randn(B, H, N, N, generator=g)
    got = []
    for fn in (reference.wkv7, cpu_ops.wkv7):
        leaves = [t.clone().requires_grad_(True) for t in ins]
        st = None if s0 is None else s0.clone().requires_grad_(True)
        y, s = fn(*leaves, N, st)
        grads = torch.autograd.grad([y, s], leaves + ([st] if st is not None else []), [dy, ds])
        got.append((y.detach(), s.detach()) + grads)
    for name, want, have in zip("y s dr dw dk dv da db ds0".split(), *got):
        assert have.dtype == want.dtype and have.shape == want.shape
        assert float((want - have).abs().max()) <= 3e-6 * float(want.abs().max()) + 1e-7, name
    with torch.no_grad():
        y, s = cpu_ops.wkv7(*ins, N, s0)
    assert torch.allclose(y, got[0][0], atol=5e-6) and torch.allclose(s, got[0][1], atol=5e-6)
    if s0 is not None:
        assert not torch.equal(s, s0) and s.data_ptr() != s0.data_ptr()              # the caller's state is left alone


def test_low_precision_inputs_get_gradients_of_their_own_dtype_and_partial_requires_grad(form):
    ins, s0 = _inputs(1, 6, 2, 8, dtype=torch.bfloat16)
    leaves = [t.clone().requires_grad_(i % 2 == 0) for i, t in enumerate(ins)]
    y, s = cpu_ops.wkv7(*leaves, 8, s0)
    assert y.dtype == torch.float32 and s.dtype == torch.float32
    (y.sum() + s.sum()).backward()
    assert all((t.grad is not None and t.grad.dtype == torch.bfloat16) == (i % 2 == 0) for i, t in enumerate(leaves))


def test_dispatch_uses_the_node_for_cpu_tensors_and_keeps_the_contract(form):
    ins, s0 = _inputs(2, 5, 2, 8)
    leaves = [t.clone().requires_grad_(True) for t in ins]
    y, s = ops.wkv7(*leaves, 8, s0, True)
    assert type(y.grad_fn).__name__ == ("_WKV7NativeBackward" if form == "native" else "_WKV7Backward")
    assert s.shape == (2, 2, 8, 8)
    y2, none = ops.wkv7(*ins, 8)
    assert none is None and torch.allclose(y2, reference.wkv7(*ins, 8)[0], atol=1e-6)


def test_norm_and_adamw_match_the_plain_statements():
    g = torch.Generator().manual_seed(0)
    grad = torch.randn(10007, generator=g)
    want = (grad * 0.25).square().sum()
    assert float(cpu_ops.grad_norm_sq(grad, 0.25)) == pytest.approx(float(want), rel=1e-5)
    assert float(cpu_ops.grad_norm_sq(grad.to(torch.bfloat16), 0.25)) == pytest.approx(
        float((grad.to(torch.bfloat16).float() * 0.25).square().sum()), rel=1e-5)
    p = torch.randn(10007, generator=g)
    state_a = [p.clone(), torch.zeros(10007), torch.zeros(10007)]
    state_b = [p.clone(), torch.zeros(10007), torch.zeros(10007)]
    scratch = torch.empty(10007)
    for step in (1, 2, 3):
        grad = torch.randn(10007, generator=g)
        reference.adamw_step(state_a[0], grad, state_a[1], state_a[2], 1e-2, 0.9, 0.99, 1e-8, 0.01, step, 0.5)
        cpu_ops.adamw_step(state_b[0], grad, state_b[1], state_b[2], 1e-2, 0.9, 0.99, 1e-8, 0.01, step, 0.5, scratch)
    for x, y in zip(state_a, state_b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-7)
    cpu_ops.adamw_step(state_b[0], grad, state_b[1], state_b[2], 1e-2, 0.9, 0.99, 1e-8, 0.01, 4, 0.5, None)      # no scratch
    assert torch.isfinite(state_b[0]).all()


def test_cpu_training_is_bit_reproducible(form):
    """Heads are independent work items, so the thread schedule cannot change a sum: same seed, same bits."""
    from rwkvtune_b200.engine import EngineConfig, TrainEngine
    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.parallel import DistContext

    def run():
        torch.manual_seed(0)
        model = RWKV7Model(RWKVConfig(n_layer=2, n_embd=128, vocab_size=256, dim_att_lora=16, dim_gate_lora=16, dim_mv_lora=16))
        eng = TrainEngine(model, EngineConfig(lr_init=1e-3, precision="fp32"), DistContext())
        g = torch.Generator().manual_seed(1)
        losses = []
        for _ in range(3):
            idx = torch.randint(0, 256, (2, 40), generator=g)
            losses.append(float(eng.train_step(idx, idx.roll(-1, 1), 1e-3)))
        return losses, eng.space.params.clone()

    (la, pa), (lb, pb) = run(), run()
    assert la == lb and torch.equal(pa, pb)
