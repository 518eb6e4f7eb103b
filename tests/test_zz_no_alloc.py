"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some users of this library cannot allocate device memory where they need a kernel (allocator
hooks, stream host callbacks, serving loops with a frozen memory plan, embedders that forbid
cudaMalloc after start-up).  For them ``rwkv_layer_norm_backward_noalloc`` keeps its scratch in a
fixed 1 MiB device array inside the library.  This test checks it against the ordinary entry
point (whose scratch the caller allocates) on two consecutive calls, because the shared array
keeps the previous call's contents, and checks that an oversized request is refused.

The file name sorts last so that a run stopping at the first failure has already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _run_both(lib, rows, C, strip, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, C, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, C, device="cuda", generator=g).to(torch.bfloat16)
    w = 1 + 0.1 * torch.randn(C, device="cuda", generator=g)
    xf = x.float()
    mean = xf.mean(-1).contiguous()
    rstd = (xf.var(-1, unbiased=False) + 1e-5).rsqrt().contiguous()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    nblocks = (rows + strip - 1) // strip

    dx_ref = torch.empty_like(x)
    partials = torch.empty(nblocks, 2, C, device="cuda", dtype=torch.float32)
    fn = lib.rwkv_layer_norm_backward
    fn.restype = ctypes.c_int
    assert fn(_ptr(dy), _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), _ptr(dx_ref), _ptr(partials), rows, C, strip,
              stream) == 0
    dw_ref, db_ref = partials.sum(0)

    dx = torch.empty_like(x)
    dw = torch.empty(C, device="cuda", dtype=torch.float32)
    db = torch.empty(C, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    fn2 = lib.rwkv_layer_norm_backward_noalloc
    fn2.restype = ctypes.c_int
    assert fn2(_ptr(dy), _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), _ptr(dx), _ptr(dw), _ptr(db), rows, C, strip,
               stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.equal(dx, dx_ref)
    scale_w, scale_b = dw_ref.abs().mean().item(), db_ref.abs().mean().item()
    assert torch.allclose(dw, dw_ref, rtol=3e-2, atol=3e-2 * scale_w + 1e-3)
    assert torch.allclose(db, db_ref, rtol=3e-2, atol=3e-2 * scale_b + 1e-3)


def test_noalloc_layer_norm_backward_matches_ordinary_entry_point():
    from rwkvtune_b200.ops import _ext

    lib = ctypes.CDLL(_ext.lib_path())
    _run_both(lib, rows=300, C=512, strip=8, seed=1)     # 38 blocks
    _run_both(lib, rows=77, C=1024, strip=4, seed=2)     # second call reuses the same scratch, other shape


def test_noalloc_rejects_oversized_request():
    from rwkvtune_b200.ops import _ext

    lib = ctypes.CDLL(_ext.lib_path())
    fn = lib.rwkv_layer_norm_backward_noalloc
    fn.restype = ctypes.c_int
    rows, C, strip = 4096, 2048, 1   # 4096 * 2 * 2048 floats = 64 MiB > 1 MiB
    null = ctypes.c_void_p(0)
    assert fn(null, null, null, null, null, null, null, null, rows, C, strip, null) == 3
