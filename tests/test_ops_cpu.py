"""CPU statements of the fused operator entry points: each must equal the composition of plain PyTorch ops it
replaces (the CUDA kernels are tested against the same statements in the GPU tests)."""
import torch
import torch.nn.functional as F

from rwkvtune_b200 import ops
from rwkvtune_b200.ops import reference as ref


def _rand(*shape, scale=0.5):
    return torch.randn(*shape) * scale


def test_gemm_entry_points_match_composition():
    torch.manual_seed(0)
    x, w, res = _rand(2, 5, 16), _rand(24, 16), _rand(2, 5, 24)
    assert torch.allclose(ops.linear(x, w), F.linear(x, w))
    assert torch.allclose(ops.linear_add(x, w, res), res + F.linear(x, w))
    assert torch.allclose(ops.linear_relu_sq(x, w), torch.relu(F.linear(x, w)) ** 2)
    w_in = _rand(16, 8)
    assert torch.allclose(ops.matmul(x, w_in), x @ w_in)
    assert torch.allclose(ops.matmul_act(x, w_in, "tanh"), torch.tanh(x @ w_in))
    assert torch.allclose(ops.matmul_act(x, w_in, "sigmoid"), torch.sigmoid(x @ w_in))
    outs = ops.linear_group([x, x * 2], [w, w[:8]])
    assert torch.allclose(outs[0], F.linear(x, w)) and torch.allclose(outs[1], F.linear(x * 2, w[:8]))
    wk, wv, r2 = _rand(64, 16), _rand(16, 64), _rand(2, 5, 16)
    assert torch.allclose(ops.channel_mix_ffn(x, wk, wv, r2), r2 + F.linear(torch.relu(F.linear(x, wk)) ** 2, wv), atol=1e-6)


def test_ln_shift_mix_unbound_returns_outputs_and_passthrough():
    torch.manual_seed(1)
    x = _rand(2, 7, 64).requires_grad_(True)
    ln_w, ln_b, mix, prev = torch.rand(64) + 0.5, _rand(64, scale=0.1), torch.rand(6, 64), _rand(2, 64)
    outs, last, x_res = ops.ln_shift_mix_unbound(x, ln_w, ln_b, mix, prev)
    stacked, last_ref = ref.ln_shift_mix(x, ln_w, ln_b, mix, prev)
    assert len(outs) == 6 and all(torch.allclose(o, s) for o, s in zip(outs, stacked.unbind(0)))
    assert torch.allclose(last, last_ref)
    # the residual connection through the returned x reaches x.grad together with the normalisation branch
    (outs[0].sum() + (x_res * 2).sum()).backward()
    g_total = x.grad.clone()
    x.grad = None
    ref.ln_shift_mix(x, ln_w, ln_b, mix, prev)[0][0].sum().backward()
    assert torch.allclose(g_total, x.grad + 2)


def test_wkv7_gn_and_pool_step_match_composition():
    torch.manual_seed(2)
    B, T, H = 2, 6, 2
    C = H * 64
    r, w, k, v, a, b = (_rand(B, T, C, scale=0.3) for _ in range(6))
    w = -F.softplus(-w) - 0.5
    g, gn_w, gn_b, r_k = torch.sigmoid(_rand(B, T, C)), torch.rand(C) + 0.5, _rand(C, scale=0.1), _rand(H, 64, scale=0.1)
    s0 = _rand(B, H, 64, 64, scale=0.1)
    z, sT = ops.wkv7_gn(r, w, k, v, a, b, g, gn_w, gn_b, r_k, 64, state=s0, return_state=True)
    y_ref, s_ref = ref.wkv7(r, w, k, v, a, b, 64, s0)
    assert torch.allclose(z, ref.gn_bonus_gate(y_ref, r, k, v, g, gn_w, gn_b, r_k, 64), atol=1e-5)
    assert torch.allclose(sT, s_ref, atol=1e-6)
    pool = _rand(5, H, 64, 64, scale=0.1)
    before, slots = pool.clone(), torch.tensor([3, 1])
    y = ops.wkv7_pool_step(r, w, k, v, a, b, pool, slots)
    y2, s2 = ref.wkv7(r, w, k, v, a, b, 64, before.index_select(0, slots))
    assert torch.allclose(y, y2, atol=1e-6) and torch.allclose(pool[slots], s2, atol=1e-6)
    assert torch.equal(pool[[0, 2, 4]], before[[0, 2, 4]])
    z2, st = ops.wkv7_gn(r, w, k, v, a, b, g, gn_w, gn_b, r_k, 64, state=(before.clone(), slots))
    assert isinstance(st, tuple) and torch.allclose(z2, ref.gn_bonus_gate(y2, r, k, v, g, gn_w, gn_b, r_k, 64), atol=1e-5)


def test_embedding_and_gather_rows():
    torch.manual_seed(3)
    table, idx = _rand(50, 16), torch.randint(0, 50, (3, 9))
    assert torch.equal(ops.embedding(idx, table), F.embedding(idx, table))
    sel = torch.tensor([4, 4, 0, 49])
    assert torch.equal(ops.gather_rows(table, sel), table.index_select(0, sel))


def test_gemm_wrappers_fall_back_on_cpu():
    """On CPU tensors the GEMM wrappers are the plain products and the split-K planner declines."""
    import torch
    from rwkvtune_b200.ops import gemm, gemm_native
    torch.manual_seed(0)
    a, b = torch.randn(40, 6), torch.randn(40, 10)
    assert gemm_native.splitk_plan(a.bfloat16(), b.bfloat16()) == 0
    assert torch.allclose(gemm.mm_tn(a, b), a.t() @ b)
    y = torch.ones(6, 10)
    assert gemm.addmm_tn_(y, a, b) is y and torch.allclose(y, 1 + a.t() @ b, atol=1e-5)
    x, w = torch.randn(5, 6), torch.randn(7, 6)
    assert torch.allclose(gemm.mm_nt(x, w), x @ w.t()) and torch.allclose(gemm.mm_nn(x, w.t().contiguous()), x @ w.t())


def test_cached_fp32_parameter_copies_refresh_together_after_an_optimiser_step():
    """The fp32 copies of small parameters are cached; after the parameters were rewritten behind autograd's back
    (the optimiser kernels write through raw pointers) one multi-tensor copy brings every cached copy up to date."""
    import torch

    from rwkvtune_b200.ops import cuda_ops

    params = [torch.nn.Parameter(torch.randn(1, 1, 16).to(torch.bfloat16)) for _ in range(5)]
    first = [cuda_ops._f32(p) for p in params]
    assert all(c.dtype == torch.float32 and torch.equal(c, p.detach().reshape(-1).float()) for c, p in zip(first, params))
    assert all(cuda_ops._f32(p) is c for p, c in zip(params, first))          # cached: same storage
    with torch.no_grad():
        for p in params:
            p.data.add_(1.0)            # .data: no version bump, as with a raw-pointer write
    assert torch.equal(cuda_ops._f32(params[0]), first[0])                     # stale until told
    cuda_ops.bump_param_epoch()
    again = cuda_ops._f32(params[0])                                           # refreshes all five at once
    assert again is first[0]
    for p, c in zip(params, first):
        assert torch.equal(c, p.detach().reshape(-1).float())
        key = (p.data_ptr(), p.numel(), p.dtype)
        assert cuda_ops._F32_CACHE[key][0] == (cuda_ops._PARAM_EPOCH, p._version)
    del params, first, again
    import gc

    gc.collect()
    cuda_ops.bump_param_epoch()
    live = torch.nn.Parameter(torch.randn(8).to(torch.bfloat16))
    cuda_ops._f32(live)
    cuda_ops.bump_param_epoch()
    cuda_ops._f32(live)                                                        # dead entries are dropped on refresh
    assert all(ref_() is not None for _, _, ref_ in cuda_ops._F32_CACHE.values())
