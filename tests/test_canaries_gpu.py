"""Guard words around kernel outputs: a kernel that writes one element outside its output (a tail tile, a ragged
row, a last partial vector) changes a canary.  The C entry points are called directly so that the output pointer
can sit inside a larger, pattern-filled allocation."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
GUARD = 4096      # elements on each side


def _guarded(numel, dtype):
    """Returns (whole buffer, output view) with ``GUARD`` pattern elements before and after the view."""
    whole = torch.empty(numel + 2 * GUARD, dtype=dtype, device="cuda")
    whole.view(torch.uint8).fill_(0x5A)
    return whole, whole[GUARD:GUARD + numel]


def _intact(whole, numel):
    raw = whole.view(torch.uint8)
    es = whole.element_size()
    return bool((raw[:GUARD * es] == 0x5A).all()) and bool((raw[(GUARD + numel) * es:] == 0x5A).all())


@pytest.mark.parametrize("M,N,K", [(136, 72, 40), (264, 264, 96), (392, 520, 200)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_tail_tiles_stay_inside_c(M, N, K, layout):
    from rwkvtune_b200.ops import _ext, gemm_native
    torch.manual_seed(0)
    if layout == "nt":
        a, b, a_mn, b_mn = torch.randn(M, K), torch.randn(N, K), 0, 0
        ref = a @ b.t()
    elif layout == "nn":
        a, b, a_mn, b_mn = torch.randn(M, K), torch.randn(K, N), 0, 1
        ref = a @ b
    else:
        a, b, a_mn, b_mn = torch.randn(K, M), torch.randn(K, N), 1, 1
        ref = a.t() @ b
    a, b = a.cuda().to(BF), b.cuda().to(BF)
    whole, c = _guarded(M * N, BF)
    c = c.view(M, N)
    _ext.call("rwkv_gemm_bf16_tcgen05", _ext.ptr(a), _ext.ptr(b), _ext.ptr(c), _ext.i32(M), _ext.i32(N), _ext.i32(K),
              _ext.i64(a.stride(0)), _ext.i64(b.stride(0)), _ext.i64(N), _ext.i32(a_mn), _ext.i32(b_mn), _ext.i32(0),
              _ext.ptr(gemm_native._status(a.device)), _ext.ptr(None), _ext.i64(0), _ext.stream())
    torch.cuda.synchronize()
    assert gemm_native.check_status() == 0
    assert _intact(whole, M * N)
    want = (a.float() @ b.float().t()) if layout == "nt" else ((a.float() @ b.float()) if layout == "nn" else a.float().t() @ b.float())
    assert (c.float() - want).abs().max() <= 2e-2 * want.abs().max() + 1e-2


@pytest.mark.parametrize("rows,C", [(37, 256), (130, 2048), (5, 768)])
def test_layer_norm_rows_stay_inside_outputs(rows, C):
    from rwkvtune_b200.ops import _ext
    torch.manual_seed(1)
    x = torch.randn(rows, C, device="cuda").to(BF)
    w, b = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda")
    wy, y = _guarded(rows * C, BF)
    wm, mean = _guarded(rows, torch.float32)
    wr, rstd = _guarded(rows, torch.float32)
    strip = 8
    _ext.call("rwkv_layer_norm_forward", _ext.ptr(x), _ext.ptr(w), _ext.ptr(b), _ext.ptr(y), _ext.ptr(mean), _ext.ptr(rstd),
              _ext.i32(rows), _ext.i32(C), _ext.i32(strip), _ext.f32(1e-5), _ext.stream())
    dy = torch.randn(rows, C, device="cuda").to(BF)
    wdx, dx = _guarded(rows * C, BF)
    n_part = -(-rows // strip) * 2 * C
    wp, partials = _guarded(n_part, torch.float32)
    _ext.call("rwkv_layer_norm_backward", _ext.ptr(dy), _ext.ptr(x), _ext.ptr(mean), _ext.ptr(rstd), _ext.ptr(w),
              _ext.ptr(dx), _ext.ptr(partials), _ext.i32(rows), _ext.i32(C), _ext.i32(strip), _ext.stream())
    torch.cuda.synchronize()
    for whole, n in ((wy, rows * C), (wm, rows), (wr, rows), (wdx, rows * C), (wp, n_part)):
        assert _intact(whole, n)
    want = torch.nn.functional.layer_norm(x.float(), (C,), w, b)
    assert (y.view(rows, C).float() - want).abs().max() < 5e-2


def test_gather_reduce_and_panel_kernels_stay_inside_outputs():
    from rwkvtune_b200.ops import _ext
    torch.manual_seed(2)
    arr = lambda ts: (ctypes.c_ulonglong * len(ts))(*[t.data_ptr() for t in ts])
    st = _ext.stream()
    # row gather with a ragged index list
    src = torch.randn(50, 40, device="cuda").to(BF)          # 80-byte rows (16-byte multiple)
    idx = torch.tensor([3, 49, 0, 17, 17, 2, 31], device="cuda")
    wo, out = _guarded(idx.numel() * 40, BF)
    _ext.call("rwkv_gather_rows", _ext.ptr(src), _ext.ptr(idx), _ext.ptr(out), _ext.i64(idx.numel()), _ext.i64(50),
              _ext.i64(80), st)
    # bucket reduce over 3 emulated ranks, 8-element granularity, few blocks
    W, lo, n = 3, 24, 1000 * 8
    grads = [torch.randn(lo + n + 64, device="cuda").to(BF) for _ in range(W)]
    wr, red = _guarded(n, torch.float32)
    wp, part = _guarded(1024, torch.float32)
    _ext.call("rwkv_zero2_reduce_bucket", arr(grads), _ext.i32(W), _ext.i64(lo), _ext.i64(n), _ext.f32(1.0), _ext.ptr(red),
              _ext.ptr(part), _ext.i32(3), _ext.i32(0), _ext.ptr(None), st)
    # panel gather and panel reduce with a row count that is not a multiple of anything convenient
    N, K, Wp = 33, 192, 3
    Kp = K // Wp
    full = torch.randn(N, K, device="cuda").to(BF)
    panels = [full[:, p * Kp:(p + 1) * Kp].contiguous() for p in range(Wp)]
    ws, staged = _guarded(N * K, BF)
    _ext.call("rwkv_ag_gather", arr(panels), _ext.i32(1), _ext.i32(Wp), _ext.i32(N), _ext.i32(K), _ext.ptr(staged),
              _ext.i32(5), st)
    dws = [torch.randn(N, K, device="cuda").to(BF) for _ in range(Wp)]
    wg, gout = _guarded(N * Kp, torch.float32)
    _ext.call("rwkv_zero3_reduce_panel", arr(dws), _ext.i32(2), _ext.i32(Wp), _ext.i32(N), _ext.i32(K), _ext.f32(1.0),
              _ext.ptr(gout), _ext.ptr(None), _ext.i32(2), _ext.i32(0), _ext.ptr(None), st)
    torch.cuda.synchronize()
    assert _intact(wo, idx.numel() * 40) and torch.equal(out.view(-1, 40), src[idx])
    assert _intact(wr, n) and _intact(wp, 1024)
    assert torch.allclose(red, sum(g[lo:lo + n].float() for g in grads), atol=1e-5)
    assert _intact(ws, N * K) and torch.equal(staged.view(N, K), full)
    assert _intact(wg, N * Kp)
    assert torch.allclose(gout.view(N, Kp), sum(d[:, 2 * Kp:3 * Kp].float() for d in dws), atol=1e-5)
