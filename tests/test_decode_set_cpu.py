"""The grouping logic of the decode path, on the CPU: which products go into which launch, with which activation,
scale and residual, is host-side code; here the kernel is replaced by a plain-PyTorch stand-in with the same contract."""
import pytest
import torch

from rwkvtune_b200.ops import gemm


class _FakeNative:
    """Stand-in for ``ops.gemm_native`` that implements ``decode_group`` with fp32 tensor math and records its calls."""
    DECODE_DISPATCH = True
    DECODE_MAX_PROBLEMS = 12

    def __init__(self, second_stage_ok=True):
        self.calls = []
        self.second_stage_ok = second_stage_ok

    def decode_ok(self, x, w, kn=False):
        if not self.second_stage_ok and self.calls:      # refuse everything after the first launch
            return False
        K = w.shape[0] if kn else w.shape[1]
        return x.dim() == 2 and x.shape[1] == K and x.shape[0] <= 128

    def decode_group(self, xs, ws, epis=None, kn=None, residuals=None, split=0, trace=None, alphas=None, res_first=None,
                     outs=None, prefetch=None):
        n = len(xs)
        kn = kn or [False] * n
        epis = epis or [None] * n
        act = {None: lambda t: t, "relu_sq": lambda t: torch.relu(t) ** 2, "tanh": torch.tanh, "sigmoid": torch.sigmoid}
        self.calls.append({"n": n, "prefetch": prefetch, "epis": list(epis), "kn": list(kn)})
        ys = []
        for i in range(n):
            y = xs[i].float() @ (ws[i].float() if kn[i] else ws[i].float().t())
            y = y * (1.0 if alphas is None or alphas[i] is None else alphas[i])
            r = None if residuals is None else residuals[i]
            if r is not None and res_first is not None and res_first[i]:
                y = act[epis[i]](y + r.float())
            else:
                y = act[epis[i]](y)
                if r is not None:
                    y = y + r.float()
            y = y.to(xs[i].dtype)
            if outs is not None and outs[i] is not None:
                outs[i].copy_(y)
                y = outs[i]
            ys.append(y)
        return ys


@pytest.fixture
def fake(monkeypatch):
    f = _FakeNative()
    monkeypatch.setattr(gemm, "_native", lambda: f)
    return f


def _rand(*shape, s=0.3):
    return (torch.randn(*shape) * s).to(torch.bfloat16)


def _close(got, want, tol=3e-2):
    return (got.float() - want.float()).abs().max().item() <= tol * max(1.0, want.float().abs().max().item())


def test_plain_set_is_one_launch_with_prefetch_hint(fake):
    torch.manual_seed(0)
    x1, x2 = _rand(5, 1, 32), _rand(5, 1, 32)
    w1, w2, res = _rand(48, 32), _rand(16, 32), _rand(5, 1, 48)
    hint = [_rand(8, 8)]
    with torch.no_grad():
        lin, low = gemm.decode_projection_set([(x1, w1, None, res, None), (x2, w2, "relu_sq", None, None)], (), hint)
    assert len(fake.calls) == 1 and fake.calls[0]["n"] == 2 and fake.calls[0]["prefetch"] is hint and low == []
    assert _close(lin[0], x1.float() @ w1.float().t() + res.float())
    assert _close(lin[1], torch.relu(x2.float() @ w2.float().t()) ** 2)
    assert lin[0].shape == (5, 1, 48)


def test_adapters_and_chains_take_two_launches(fake):
    torch.manual_seed(1)
    M, C, r, d = 6, 32, 8, 16
    x, xk, xw = _rand(M, 1, C), _rand(M, 1, C), _rand(M, 1, C)
    W, A, B = _rand(C, C), _rand(r, C), _rand(C, r)
    Wk, Ak, Bk = _rand(2 * C, C), _rand(r, C), _rand(2 * C, r)
    w1, w2 = _rand(C, d), _rand(d, C)
    res = _rand(M, 1, C)
    s = 1.7
    with torch.no_grad():
        lin, low = gemm.decode_projection_set(
            [(x, W, None, res, (A, B, s)), (xk, Wk, "relu_sq", None, (Ak, Bk, s))], [(xw, w1, "tanh", w2)])
    # first launch: two base products, two x A^T, one chain first stage; second: two B products in place, one second stage
    assert [c["n"] for c in fake.calls] == [5, 3]
    assert fake.calls[0]["epis"] == [None, None, None, None, "tanh"] and fake.calls[0]["kn"] == [False] * 4 + [True]
    assert fake.calls[1]["epis"] == [None, "relu_sq", None]
    f32 = lambda *ts: [t.float() for t in ts]
    x_, xk_, xw_, W_, A_, B_, Wk_, Ak_, Bk_, w1_, w2_, res_ = f32(x, xk, xw, W, A, B, Wk, Ak, Bk, w1, w2, res)
    want0 = x_ @ W_.t() + s * (x_ @ A_.t()) @ B_.t() + res_
    want1 = torch.relu(xk_ @ Wk_.t() + s * (xk_ @ Ak_.t()) @ Bk_.t()) ** 2
    assert _close(lin[0], want0) and _close(lin[1], want1)
    assert _close(low[0], torch.tanh(xw_ @ w1_) @ w2_)


def test_second_launch_refused_falls_back_to_plain_products(monkeypatch):
    f = _FakeNative(second_stage_ok=False)
    monkeypatch.setattr(gemm, "_native", lambda: f)
    torch.manual_seed(2)
    M, C, r, d = 4, 16, 8, 8
    x, xw = _rand(M, C), _rand(M, C)
    W, A, B = _rand(C, C), _rand(r, C), _rand(C, r)
    w1, w2 = _rand(C, d), _rand(d, C)
    with torch.no_grad():
        lin, low = gemm.decode_projection_set([(x, W, "relu_sq", None, (A, B, 0.5))], [(xw, w1, None, w2)])
    assert len(f.calls) == 1
    x_, xw_, W_, A_, B_, w1_, w2_ = (t.float() for t in (x, xw, W, A, B, w1, w2))
    assert _close(lin[0], torch.relu(x_ @ W_.t() + 0.5 * (x_ @ A_.t()) @ B_.t()) ** 2)
    assert _close(low[0], (xw_ @ w1_) @ w2_)


def test_set_does_not_apply_while_autograd_records_or_with_too_many_problems(fake):
    x, w = _rand(3, 8), _rand(8, 8)
    assert gemm.decode_projection_set([(x, w, None, None, None)]) is None          # grad mode on
    with torch.no_grad():
        assert gemm.decode_projection_set([(x, w, None, None, None)] * 13) is None
        # an activation together with a residual cannot be combined with an adapter in two launches
        assert gemm.decode_projection_set([(x, w, "relu_sq", _rand(3, 8), (_rand(4, 8), _rand(8, 4), 1.0))]) is None
    assert fake.calls == []


def test_decode_order_links_are_plain_attributes_not_submodules():
    """Each half of a block knows which half runs next (for the L2 prefetch hints of the decode path); the links must
    not show up as sub-modules, parameters or state-dict entries, and the model must still deep-copy."""
    import copy

    from rwkvtune_b200.models import RWKVConfig, RWKV7Model
    from rwkvtune_b200.models.rwkv7.model import _weights_of

    m = RWKV7Model(RWKVConfig(n_layer=3, n_embd=64, vocab_size=128))
    for i, blk in enumerate(m.blocks):
        assert blk.att._decode_next is blk.ffn
        assert blk.ffn._decode_next is (m.blocks[i + 1].att if i + 1 < 3 else None)
    names = [n for n, _ in m.named_modules()]
    assert not any("_decode_next" in n for n in names) and len(names) == len(set(names))
    assert not any("_decode_next" in k for k in m.state_dict())
    n_params = sum(1 for _ in m.parameters())
    m2 = copy.deepcopy(m)
    assert sum(1 for _ in m2.parameters()) == n_params
    assert m2.blocks[0].att._decode_next is m2.blocks[0].ffn          # the copy links to its own halves
    assert _weights_of(m.blocks[0].ffn.key, None) == []                # CPU weights give no hint


def test_launch_chaining_and_capture_guard_are_inert_without_a_gpu():
    import gc

    from rwkvtune_b200.ops import _ext

    with _ext.launch_chaining():
        assert _ext.chaining() is False or _ext.available()
    was = gc.isenabled()
    with _ext.capture_safe_gc():
        assert not gc.isenabled()
    assert gc.isenabled() == was
