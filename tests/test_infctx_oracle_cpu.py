"""The closed-form WKV7 backward (reverse recurrence with state gradient) against autograd of the fp32 recurrence."""
import pytest
import torch

from rwkvtune_b200.models.rwkv7 import operators as O
from rwkvtune_b200.ops import reference


def _inputs(B=2, T=7, H=2, N=8, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=dtype)
    q, k, v = rnd(B, T, H, N), rnd(B, T, H, N) * 0.5, rnd(B, T, H, N)
    w = -0.5 - torch.rand(B, T, H, N, generator=g, dtype=dtype)          # raw decay input; d = exp(-exp(w))
    kk = torch.nn.functional.normalize(rnd(B, T, H, N), dim=-1)
    a, b = -kk, kk * torch.rand(B, T, H, N, generator=g, dtype=dtype)
    s0 = rnd(B, H, N, N) * 0.3
    return q, k, v, w, a, b, s0


def _autograd(q, k, v, w, a, b, s0, scale, dy, ds):
    B, T, H, N = q.shape
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v, w, a, b)]
    s = None if s0 is None else s0.float().clone().requires_grad_(True)
    flat = lambda t: t.reshape(B, T, H * N)
    y, s1 = reference.wkv7(flat(leaves[0] * scale), flat(leaves[3]), flat(leaves[1]), flat(leaves[2]), flat(leaves[4]),
                           flat(leaves[5]), N, s)
    targets = leaves + ([s] if s is not None else [])
    grads = torch.autograd.grad([y.reshape(B, T, H, N), s1], targets, [dy.float(), ds.float()])
    return y.reshape(B, T, H, N), s1, grads


@pytest.mark.parametrize("with_state,scale", [(True, 1.0), (False, 0.5), (True, 0.125)])
def test_closed_form_backward_matches_autograd(with_state, scale):
    q, k, v, w, a, b, s0 = _inputs()
    s0 = s0 if with_state else None
    g = torch.Generator().manual_seed(1)
    dy = torch.randn(q.shape, generator=g)
    ds = torch.randn(q.shape[0], q.shape[2], q.shape[3], q.shape[3], generator=g)
    y_ref, s_ref, g_ref = _autograd(q, k, v, w, a, b, s0, scale, dy, ds)
    y, s1 = O.naive_recurrent_rwkv7_fwd(q, k, v, w, a, b, scale, s0)
    assert y.dtype == torch.float32 and torch.allclose(y, y_ref, atol=1e-5) and torch.allclose(s1, s_ref, atol=1e-5)
    grads = O.naive_recurrent_rwkv7_bwd(q, k, v, w, a, b, dy, ds, scale, s0)
    assert len(grads) == 7
    for name, got, want in zip("q k v w a b s0".split(), grads, g_ref):
        err = (got - want).abs().max() / want.abs().max().clamp_min(1e-6)
        assert err < 2e-5, (name, float(err))


def test_functions_carry_state_gradient_across_two_chunks():
    """Two chunks chained through the state give the gradients of one pass over the whole sequence: through the
    closed-form function, and through the wrapper of the chunk-step operator."""
    q, k, v, w, a, b, s0 = _inputs(T=8, dtype=torch.float32)
    g = torch.Generator().manual_seed(2)
    dy = torch.randn(q.shape, generator=g)
    ds = torch.zeros_like(s0)
    _, _, g_ref = _autograd(q, k, v, w, a, b, s0, 1.0, dy, ds)

    def chained(step):
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, w, a, b)]
        s = s0.clone().requires_grad_(True)
        y1, mid = step(*(t[:, :5] for t in leaves), s)
        y2, _ = step(*(t[:, 5:] for t in leaves), mid)
        return torch.autograd.grad(torch.cat([y1, y2], 1), leaves + [s], dy)

    naive = chained(lambda q_, k_, v_, w_, a_, b_, s: O.RWKV7InfctxNaiveFunction.apply(q_, k_, v_, w_, a_, b_, 1.0, s))
    wrapped = chained(lambda q_, k_, v_, w_, a_, b_, s: O.WKV7InfctxFunction.apply(w_, q_, k_, v_, a_, b_, s))
    for got in (naive, wrapped):
        for name, x, want in zip("q k v w a b s0".split(), got, g_ref):
            assert torch.allclose(x, want, atol=2e-5, rtol=1e-4), name


def test_no_initial_state_returns_no_state_gradient():
    q, k, v, w, a, b, _ = _inputs(T=4, dtype=torch.float32)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, w, a, b)]
    y, s1 = O.rwkv7_wkv_infctx_naive(*leaves)
    (y.sum() + s1.sum()).backward()
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in leaves)
