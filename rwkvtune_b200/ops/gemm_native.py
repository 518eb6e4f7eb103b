"""Binding of the tcgen05 GEMM (``rwkvtune_b200/csrc/gemm_tcgen05.cu``).

``native_ok`` states which problems the kernel takes: bf16 CUDA tensors, 16-byte aligned rows
(every leading dimension a multiple of 8 elements) and sizes large enough that a 128x256 tile is
not mostly padding.  Weight-gradient products with few output tiles and a long contraction take the kernel's
split-K path (``splitk_plan`` / ``mm_tn_splitk``).  Everything else goes to the library GEMM.
"""
from __future__ import annotations

import torch

from . import _ext

_STATUS = {}
MIN_M, MIN_N, MIN_K = 128, 64, 32


def _status(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device=None) -> int:
    """Host-side read of the device status word (non-zero = a bounded wait inside the kernel expired)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_status(dev).item())


_STATUS_HOST = {}


def check_status_nosync(device=None) -> int:
    """Status word as of the last :func:`snapshot_status` (a pinned host copy: no device synchronisation)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    host = _STATUS_HOST.get(key)
    return 0 if host is None else int(host[0])


def snapshot_status(device=None) -> None:
    """Queue an asynchronous copy of the status word to pinned host memory (call at the end of a step)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _STATUS_HOST:
        _STATUS_HOST[key] = torch.zeros(1, dtype=torch.int32).pin_memory()
    _STATUS_HOST[key].copy_(_status(dev), non_blocking=True)


_HAS_GEMM = None


def available() -> bool:
    global _HAS_GEMM
    if _HAS_GEMM is None:
        _HAS_GEMM = _ext.available() and hasattr(_ext.lib(), "rwkv_gemm_bf16_tcgen05")
    return _HAS_GEMM


def _rows_ok(t: torch.Tensor) -> bool:
    return (t.dim() == 2 and t.dtype == torch.bfloat16 and t.is_cuda and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def native_ok(x: torch.Tensor, w: torch.Tensor, layout: str) -> bool:
    if not (_rows_ok(x) and _rows_ok(w)) or not available():
        return False
    if layout == "nt":
        M, K, N = x.shape[0], x.shape[1], w.shape[0]
    elif layout == "nn":
        M, K, N = x.shape[0], x.shape[1], w.shape[1]
    else:
        M, K, N = x.shape[1], x.shape[0], w.shape[1]
    if not (M >= MIN_M and N >= MIN_N and K >= MIN_K and N % 8 == 0):
        return False
    tiles = -(-M // 128) * -(-N // 256)
    # a long contraction spread over few output tiles belongs to the split-K path (see splitk_plan)
    return tiles >= 64 or K <= 4096


def _run(a, b, M, N, K, a_mn: int, b_mn: int, epilogue: int = 0, out: torch.Tensor = None,
         residual: torch.Tensor = None, accumulate: bool = True) -> torch.Tensor:
    """``out`` given: accumulate into it (epilogue 2, ``out += op(a) op(b)``) or, with ``accumulate=False``, store
    into it.  ``residual`` given: return ``residual + op(a) op(b)`` in a new tensor.  Both must be bf16 ``[M, N]``
    with unit inner stride."""
    eff = (2 if accumulate else epilogue) if out is not None else (2 if (residual is not None and epilogue == 0) else epilogue)
    if two_cta_ok(M, N, K, eff):
        return _run_2cta(a, b, M, N, K, a_mn, b_mn, epilogue, out, residual, accumulate)
    if out is not None:
        c, epilogue = out, (2 if accumulate else epilogue)
    else:
        c = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
        if residual is not None and epilogue == 0:
            epilogue = 2
    _ext.call("rwkv_gemm_bf16_tcgen05", _ext.ptr(a), _ext.ptr(b), _ext.ptr(c), _ext.i32(M), _ext.i32(N), _ext.i32(K),
              _ext.i64(a.stride(0)), _ext.i64(b.stride(0)), _ext.i64(c.stride(0)), _ext.i32(a_mn), _ext.i32(b_mn),
              _ext.i32(epilogue), _ext.ptr(_status(a.device)), _ext.ptr(residual),
              _ext.i64(0 if residual is None else residual.stride(0)), _ext.stream())
    return c


def mm_nt(x: torch.Tensor, w: torch.Tensor, epilogue: int = 0, out: torch.Tensor = None,
          residual: torch.Tensor = None) -> torch.Tensor:
    """``x [M,K] @ w[N,K]^T``"""
    return _run(x, w, x.shape[0], w.shape[0], x.shape[1], 0, 0, epilogue, out, residual)


# The pair-of-SMs kernel (``gemm_tcgen05_2cta.cu``: 256x256 tiles, tcgen05.mma.cta_group::2) serves every layout with
# epilogues 0, 1, 2, 5 when the output has at least one 256x256 tile per SM pair; smaller products, the tanh / sigmoid
# epilogues and split-K stay on the single-CTA kernel.  Measured on the 1.5B step: 386-388 -> 367-369 ms.
TWO_CTA = __import__("os").environ.get("RWKVTUNE_GEMM_2CTA", "1") == "1"    # RWKVTUNE_GEMM_2CTA=0: single-CTA kernel only


TWO_CTA_MIN_TILES = int(__import__("os").environ.get("RWKVTUNE_GEMM_2CTA_MIN_TILES", "48"))   # of 74 SM pairs


def two_cta_ok(M: int, N: int, K: int, epilogue: int) -> bool:
    return (TWO_CTA and epilogue in (0, 1, 2, 5) and M >= 256 and N >= 256 and -(-M // 256) * -(-N // 256) >= TWO_CTA_MIN_TILES
            and hasattr(_ext.lib(), "rwkv_gemm_bf16_tcgen05_2cta"))


def _run_2cta(a, b, M, N, K, a_mn: int, b_mn: int, epilogue: int = 0, out: torch.Tensor = None,
              residual: torch.Tensor = None, accumulate: bool = True, a2: torch.Tensor = None,
              b2: torch.Tensor = None, K2: int = 0) -> torch.Tensor:
    """Same contract as :func:`_run`, on the pair-of-SMs kernel.  ``a2`` / ``b2`` (same layouts as ``a`` / ``b``,
    contraction length ``K2``) are appended to the contraction: ``op(a) op(b) + op(a2) op(b2)`` in one launch."""
    if out is not None:
        c, epilogue = out, (2 if accumulate else epilogue)
    else:
        c = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
        if residual is not None and epilogue == 0:
            epilogue = 2
    if a2 is None:
        _ext.call("rwkv_gemm_bf16_tcgen05_2cta", _ext.ptr(a), _ext.ptr(b), _ext.ptr(c), _ext.i32(M), _ext.i32(N),
                  _ext.i32(K), _ext.i64(a.stride(0)), _ext.i64(b.stride(0)), _ext.i64(c.stride(0)), _ext.i32(a_mn),
                  _ext.i32(b_mn), _ext.i32(epilogue), _ext.ptr(_status(a.device)), _ext.ptr(residual),
                  _ext.i64(0 if residual is None else residual.stride(0)), _ext.stream())
    else:
        _ext.call("rwkv_gemm_bf16_tcgen05_2cta_dual", _ext.ptr(a), _ext.ptr(b), _ext.ptr(c), _ext.i32(M), _ext.i32(N),
                  _ext.i32(K), _ext.i64(a.stride(0)), _ext.i64(b.stride(0)), _ext.i64(c.stride(0)), _ext.i32(a_mn),
                  _ext.i32(b_mn), _ext.i32(epilogue), _ext.ptr(_status(a.device)), _ext.ptr(residual),
                  _ext.i64(0 if residual is None else residual.stride(0)), _ext.ptr(a2), _ext.ptr(b2), _ext.i32(K2),
                  _ext.i64(a2.stride(0)), _ext.i64(b2.stride(0)), _ext.stream())
    return c


def dual_ok(x: torch.Tensor, w: torch.Tensor, x2: torch.Tensor, w2: torch.Tensor, layout: str) -> bool:
    """``x w^T + x2 w2^T`` (``layout="nt"``) or ``x w + x2 w2`` (``"nn"``) as one launch of the pair-of-SMs kernel."""
    if not (available() and hasattr(_ext.lib(), "rwkv_gemm_bf16_tcgen05_2cta_dual")):
        return False
    if not all(t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and _rows_ok(t) for t in (x, w, x2, w2)):
        return False
    M, K = x.shape
    N = w.shape[0] if layout == "nt" else w.shape[1]
    K2 = x2.shape[1]
    shapes = (w.shape == (N, K) and w2.shape == (N, K2)) if layout == "nt" else (w.shape == (K, N) and w2.shape == (K2, N))
    return shapes and x2.shape[0] == M and K2 > 0 and two_cta_ok(M, N, K, 0)


def mm_nt_dual(x, w, x2, w2, epilogue: int = 0, residual: torch.Tensor = None) -> torch.Tensor:
    """``x [M,K] @ w[N,K]^T + x2 [M,K2] @ w2[N,K2]^T``: the second product rides as extra K blocks of the first.
    ``epilogue=1``: relu(.)^2 of the sum; ``residual`` ([M,N] bf16): added in the epilogue."""
    return _run_2cta(x, w, x.shape[0], w.shape[0], x.shape[1], 0, 0, epilogue=epilogue, residual=residual, a2=x2, b2=w2,
                     K2=x2.shape[1])


def mm_nn_dual(x, w, x2, w2) -> torch.Tensor:
    """``x [M,K] @ w[K,N] + x2 [M,K2] @ w2[K2,N]``."""
    return _run_2cta(x, w, x.shape[0], w.shape[1], x.shape[1], 0, 1, a2=x2, b2=w2, K2=x2.shape[1])


def mm_nt_2cta(x: torch.Tensor, w: torch.Tensor, epilogue: int = 0, out: torch.Tensor = None,
               residual: torch.Tensor = None) -> torch.Tensor:
    """``x [M,K] @ w[N,K]^T`` on pairs of SMs.  ``out`` given: ``out += x w^T``; ``residual`` given: returns
    ``residual + x w^T``."""
    return _run_2cta(x, w, x.shape[0], w.shape[0], x.shape[1], 0, 0, epilogue, out, residual)


def mm_nn_2cta(x: torch.Tensor, w: torch.Tensor, epilogue: int = 0, out: torch.Tensor = None,
               residual: torch.Tensor = None) -> torch.Tensor:
    """``x [M,K] @ w[K,N]`` on pairs of SMs."""
    return _run_2cta(x, w, x.shape[0], w.shape[1], x.shape[1], 0, 1, epilogue, out, residual)


def mm_tn_2cta(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, accumulate: bool = True) -> torch.Tensor:
    """``a[Kc,M]^T @ b[Kc,N]`` on pairs of SMs."""
    return _run_2cta(a, b, a.shape[1], b.shape[1], a.shape[0], 1, 1, 0, out, None, accumulate)


def mm_nn(x: torch.Tensor, w: torch.Tensor, epilogue: int = 0, out: torch.Tensor = None,
          residual: torch.Tensor = None) -> torch.Tensor:
    """``x [M,K] @ w[K,N]``; with ``epilogue=5`` the result is multiplied by ``2 sqrt(residual)``."""
    return _run(x, w, x.shape[0], w.shape[1], x.shape[1], 0, 1, epilogue, out, residual)


def mm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, accumulate: bool = True) -> torch.Tensor:
    """``a[Kc,M]^T @ b[Kc,N]`` (weight gradients: contraction over the token dimension)"""
    return _run(a, b, a.shape[1], b.shape[1], a.shape[0], 1, 1, 0, out, None, accumulate)


_SPLITK_WS = {}
SPLITK_MIN_K = 8192


def splitk_plan(a: torch.Tensor, b: torch.Tensor) -> int:
    """Number of K slices for ``a[Kc,M]^T @ b[Kc,N]`` when it has few output tiles and a long contraction (the weight
    gradients of the low-rank maps: 8-16 tiles, Kc = tokens); 0 when the product is not of that kind."""
    if not (_rows_ok(a) and _rows_ok(b)) or not available() or not hasattr(_ext.lib(), "rwkv_gemm_bf16_tcgen05_splitk"):
        return 0
    Kc, M, N = a.shape[0], a.shape[1], b.shape[1]
    if M < 64 or N < MIN_N or N % 8 or Kc < SPLITK_MIN_K:
        return 0
    tiles = -(-M // 128) * -(-N // 256)
    if tiles >= 64:
        return 0
    splits = min(148 // tiles, -(-Kc // 64) // 8, 32)
    return splits if splits >= 2 else 0


def mm_tn_splitk(a: torch.Tensor, b: torch.Tensor, splits: int) -> torch.Tensor:
    """``a[Kc,M]^T @ b[Kc,N]`` with the contraction cut into ``splits`` slices (fp32 slice tiles + one reduce)."""
    Kc, M, N = a.shape[0], a.shape[1], b.shape[1]
    key = a.device.index
    ws = _SPLITK_WS.get(key)
    need = splits * M * N
    if ws is None or ws.numel() < need:
        ws = _SPLITK_WS[key] = torch.empty(max(need, 1 << 22), dtype=torch.float32, device=a.device)
    c = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    _ext.call("rwkv_gemm_bf16_tcgen05_splitk", _ext.ptr(a), _ext.ptr(b), _ext.ptr(c), _ext.i32(M), _ext.i32(N),
              _ext.i32(Kc), _ext.i64(a.stride(0)), _ext.i64(b.stride(0)), _ext.i64(c.stride(0)), _ext.i32(1), _ext.i32(1),
              _ext.i32(splits), _ext.ptr(ws), _ext.ptr(_status(a.device)), _ext.stream())
    return c


class GatheredWeight:
    """A ``[N, K]`` weight stored as ``world`` K-panels (one per rank) plus the local staging matrix the
    all-gather-fused GEMM fills.  ``shard_ptrs`` are device addresses of every rank's ``[N, K/world]`` panel as
    mapped in this process (symmetric memory); on one GPU they can be plain local tensors (used by tests)."""

    def __init__(self, shard_ptrs, rank: int, world: int, N: int, K: int, device, n_copy: int = 16):
        import ctypes

        self.rank, self.world, self.N, self.K = rank, world, N, K
        self.ptrs = (ctypes.c_ulonglong * world)(*[int(p) for p in shard_ptrs])
        self.staged = torch.empty(N, K, dtype=torch.bfloat16, device=device)
        self.counts = torch.zeros(world * (-(-N // 256)), dtype=torch.int32, device=device)   # per (panel, 256-row block)
        self.arrivals = ctypes.c_int(0)      # running arrival total per counter, advanced by every call


def ag_mm_nt(x: torch.Tensor, gw: GatheredWeight, x2: torch.Tensor = None, w2: torch.Tensor = None, epilogue: int = 0,
             residual: torch.Tensor = None) -> torch.Tensor:
    """``x [M,K] @ W^T`` with the all-gather of ``W`` fused into the GEMM; afterwards ``gw.staged`` holds ``W``.
    ``x2 [M,K2]`` / ``w2 [N,K2]`` (local, contiguous): ``+ x2 @ w2^T``, appended to the contraction of the same launch.
    ``epilogue=1``: relu(.)^2; ``residual [M,N]`` (bf16, local): added in the epilogue."""
    import ctypes

    M = x.shape[0]
    y = torch.empty(M, gw.N, dtype=torch.bfloat16, device=x.device)
    if gw.arrivals.value > 0x60000000:       # counters are 32-bit: start over long before they wrap
        torch.cuda.current_stream().synchronize()
        gw.counts.zero_()
        gw.arrivals.value = 0
    if residual is not None:
        epilogue = 2
    fused = (x2 is not None or epilogue) and hasattr(_ext.lib(), "rwkv_ag_gemm_bf16_tcgen05_fused")
    if (x2 is not None or epilogue) and not fused:
        raise RuntimeError("this build of the native library has no fused variant of the all-gather GEMM")
    if fused and x2 is None:
        _ext.call("rwkv_ag_gemm_bf16_tcgen05_fused", _ext.ptr(x), gw.ptrs, _ext.ptr(gw.staged), _ext.ptr(y), _ext.i32(M),
                  _ext.i32(gw.N), _ext.i32(gw.K), _ext.i32(gw.rank), _ext.i32(gw.world), _ext.ptr(gw.counts),
                  ctypes.byref(gw.arrivals), _ext.ptr(_status(x.device)), _ext.ptr(None), _ext.ptr(None), _ext.i32(0),
                  _ext.i32(epilogue), _ext.ptr(residual), _ext.i64(0 if residual is None else residual.stride(0)),
                  _ext.stream())
        return y
    if fused:
        if not (x2.is_contiguous() and w2.is_contiguous() and x2.shape == (M, w2.shape[1]) and w2.shape[0] == gw.N
                and x2.shape[1] % 8 == 0 and x2.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16):
            raise ValueError("appended operand pair must be contiguous bf16 [M, K2] and [N, K2] with K2 a multiple of 8")
        _ext.call("rwkv_ag_gemm_bf16_tcgen05_fused", _ext.ptr(x), gw.ptrs, _ext.ptr(gw.staged), _ext.ptr(y), _ext.i32(M),
                  _ext.i32(gw.N), _ext.i32(gw.K), _ext.i32(gw.rank), _ext.i32(gw.world), _ext.ptr(gw.counts),
                  ctypes.byref(gw.arrivals), _ext.ptr(_status(x.device)), _ext.ptr(x2), _ext.ptr(w2),
                  _ext.i32(x2.shape[1]), _ext.i32(epilogue), _ext.ptr(residual),
                  _ext.i64(0 if residual is None else residual.stride(0)), _ext.stream())
        return y
    _ext.call("rwkv_ag_gemm_bf16_tcgen05", _ext.ptr(x), gw.ptrs, _ext.ptr(gw.staged), _ext.ptr(y), _ext.i32(M),
              _ext.i32(gw.N), _ext.i32(gw.K), _ext.i32(gw.rank), _ext.i32(gw.world), _ext.ptr(gw.counts),
              ctypes.byref(gw.arrivals), _ext.ptr(_status(x.device)), _ext.stream())
    return y


# ------------------------------------------------------------------------------- decode GEMM (tcgen05, clusters)
import os as _os

DECODE_MAX_M = 128
# The rollout path sends its projections here (``gemm_decode_tcgen05.cu``); RWKVTUNE_DECODE_GEMM=0 leaves them on
# the library GEMM.
DECODE_DISPATCH = _os.environ.get("RWKVTUNE_DECODE_GEMM", "1") == "1"
DECODE_EPI = {None: 0, "none": 0, "relu_sq": 1, "tanh": 3, "sigmoid": 4}
_HAS_DECODE = None


def decode_available() -> bool:
    global _HAS_DECODE
    if _HAS_DECODE is None:
        _HAS_DECODE = _ext.available() and hasattr(_ext.lib(), "rwkv_gemm_decode_tcgen05")
    return _HAS_DECODE


def decode_ok(x: torch.Tensor, w: torch.Tensor, kn: bool = False) -> bool:
    """``x [M, K]`` times ``w`` (``[N, K]``, or ``[K, N]`` with ``kn``) with at most 128 rows: one grouped
    weight-streaming launch (see ``gemm_decode_tcgen05.cu``)."""
    if not (decode_available() and x.is_cuda and x.dim() == 2 and w.dim() == 2 and x.dtype == torch.bfloat16
            and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= DECODE_MAX_M and x.is_contiguous()
            and w.is_contiguous() and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return False
    K, N = (w.shape[0], w.shape[1]) if kn else (w.shape[1], w.shape[0])
    return x.shape[1] == K and K % 8 == 0 and N % 8 == 0


DECODE_MAX_PROBLEMS = 12


def decode_group(xs, ws, epis=None, kn=None, residuals=None, split: int = 0, trace=None, alphas=None, res_first=None,
                 outs=None, prefetch=None):
    """``[act_i(alpha_i * x_i @ W_i) + residual_i]`` (or ``act_i(alpha_i * x_i @ W_i + residual_i)`` where
    ``res_first[i]``) for up to 12 problems sharing the row count, in one launch.  ``kn[i]`` marks a weight stored
    ``[K, N]``; ``epis[i]`` is one of ``DECODE_EPI``; a residual is a contiguous ``[M, N_i]`` bf16 tensor and may be the
    output itself (``outs[i]``: accumulate in place).  ``trace``: optional zeroed int64 CUDA tensor of at least
    16 x (number of CTAs) entries that receives the per-CTA phase time stamps (``benchmarks/decode_gemm_timeline.py``).
    ``prefetch``: weight tensors that later launches of the step will read (the four largest are used): the kernel asks
    for them to be brought into L2 once its own tiles are requested."""
    import ctypes

    n = len(xs)
    M = xs[0].shape[0]
    kn = list(kn) if kn is not None else [False] * n
    Ns = [w.shape[1] if t else w.shape[0] for w, t in zip(ws, kn)]
    Ks = [w.shape[0] if t else w.shape[1] for w, t in zip(ws, kn)]
    ys = [o if (outs is not None and (o := outs[i]) is not None)
          else torch.empty(M, N, dtype=torch.bfloat16, device=xs[0].device) for i, N in enumerate(Ns)]
    vp = ctypes.c_void_p * n
    ip = ctypes.c_int * n
    res = None
    if residuals is not None and any(r is not None for r in residuals):
        res = vp(*[(r.data_ptr() if r is not None else None) for r in residuals])
    codes = ip(*[DECODE_EPI[e] for e in (epis if epis is not None else [None] * n)])
    al = None if alphas is None else (ctypes.c_float * n)(*[1.0 if v is None else float(v) for v in alphas])
    rf = None if res_first is None else ip(*[int(bool(v)) for v in res_first])
    args = (vp(*[t.data_ptr() for t in xs]), vp(*[t.data_ptr() for t in ws]), vp(*[t.data_ptr() for t in ys]), res,
            ip(*Ns), ip(*Ks), codes, ip(*[int(t) for t in kn]), al, rf, _ext.i32(n), _ext.i32(M), _ext.i32(split),
            _ext.i32(1 if _ext.chaining() else 0), _ext.ptr(_status(xs[0].device)), _ext.stream())
    nxt = [t for t in (prefetch or ()) if t is not None and t.is_cuda and t.numel() > 0 and t.data_ptr() % 16 == 0]
    if trace is None and not nxt:
        _ext.call("rwkv_gemm_decode_tcgen05", *args)
    else:
        nxt = sorted(nxt, key=lambda t: -t.numel())[:4]
        k = len(nxt)
        np_ = (ctypes.c_void_p * max(k, 1))(*[t.data_ptr() for t in nxt]) if k else None
        nb_ = (ctypes.c_longlong * max(k, 1))(*[t.numel() * t.element_size() for t in nxt]) if k else None
        _ext.call("rwkv_gemm_decode_tcgen05_traced", *args, _ext.ptr(trace), np_, nb_, _ext.i32(k))
    return ys
