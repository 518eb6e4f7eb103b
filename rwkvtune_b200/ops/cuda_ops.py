"""Autograd wrappers around the native sm_100a kernels.

Each public function mirrors a function of :mod:`rwkvtune_b200.ops.reference`.
Tensors handed to a kernel are made contiguous and bf16 where the kernel is bf16
only; shapes are validated here so the kernels themselves stay branch-free.
"""
from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import _ext
from . import reference as ref
from ._ext import call, f32, i32, i64, ptr, stream

BF16 = torch.bfloat16
INPLACE_STATE = False   # set by the rollout engine while decoding: WKV state tensors are updated in place


def _c(t: torch.Tensor, dtype=None) -> torch.Tensor:
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t if t.is_contiguous() else t.contiguous()


# =============================================================================== WKV7
class _WKV7(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, state, return_state: bool, track: bool = True):
        B, T, C = r.shape
        H = C // 64
        out_dtype = r.dtype
        r, w, k, v, a, b = (_c(t, BF16) for t in (r, w, k, v, a, b))
        s0 = None if state is None else _c(state, torch.float32)
        # `track` is the caller's grad mode (inside forward it is always off): under no_grad nothing is saved, even
        # when the inputs derive from parameters that require grad (rollouts with the training model)
        need_grad = track and any(ctx.needs_input_grad[:7])
        y = torch.empty(B, T, C, dtype=BF16, device=r.device)
        NC = (T + 15) // 16
        sa = torch.empty(B, T, C, dtype=torch.float32, device=r.device) if need_grad else None
        ckpt = torch.empty(B, H, NC, 64, 64, dtype=torch.float32, device=r.device) if need_grad else None
        if return_state and INPLACE_STATE and s0 is not None and not need_grad and s0.data_ptr() == state.data_ptr():
            s_final = s0        # decode: the kernel reads a head's state before it writes it, so in/out may alias
        else:
            s_final = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device) if return_state else None
        call("rwkv_wkv7_forward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(s0), ptr(y), ptr(sa),
             ptr(ckpt), ptr(s_final), i32(B), i32(T), i32(H), stream())
        if need_grad:
            ctx.save_for_backward(r, w, k, v, a, b, sa, ckpt)
        ctx.has_state = state is not None
        ctx.out_dtype = out_dtype
        ctx.shape = (B, T, H)
        y = y if out_dtype == BF16 else y.to(out_dtype)
        if return_state:
            return y, s_final
        return y, None

    @staticmethod
    def backward(ctx, dy, ds_final):
        r, w, k, v, a, b, sa, ckpt = ctx.saved_tensors
        B, T, H = ctx.shape
        dy = _c(dy, BF16)
        ds_T = None if ds_final is None else _c(ds_final, torch.float32)
        grads = [torch.empty_like(r) for _ in range(6)]
        ds0 = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device) if ctx.has_state else None
        call("rwkv_wkv7_backward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(dy), ptr(sa), ptr(ckpt),
             ptr(ds_T), *(ptr(g) for g in grads), ptr(ds0), i32(B), i32(T), i32(H), stream())
        if ctx.out_dtype != BF16:
            grads = [g.to(ctx.out_dtype) for g in grads]
        return (*grads, ds0, None, None)


def _tc_ws(B, T, H, device):
    """Chunk-product workspace of the tensor-core WKV7 kernels (10 496 bytes per 16-step chunk)."""
    return torch.empty(B * H * ((T + 15) // 16) * 10496, dtype=torch.uint8, device=device)


class _WKV7TC(torch.autograd.Function):
    """Chunked tensor-core WKV7 (16-step chunks).  Saves the bf16 state at the start of every chunk; the
    backward recomputes the intra-chunk quantities from the inputs and those states."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b, state, return_state: bool, track: bool = True):
        B, T, C = r.shape
        H = C // 64
        out_dtype = r.dtype
        r, w, k, v, a, b = (_c(t, BF16) for t in (r, w, k, v, a, b))
        s0 = None if state is None else _c(state, torch.float32)
        # `track` is the caller's grad mode (inside forward it is always off): under no_grad nothing is saved, even
        # when the inputs derive from parameters that require grad (rollouts with the training model)
        need_grad = track and any(ctx.needs_input_grad[:7])
        NC = (T + 15) // 16
        y = torch.empty(B, T, C, dtype=BF16, device=r.device)
        cs = torch.empty(B, H, NC, 64, 64, dtype=BF16, device=r.device) if need_grad else None
        s_final = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device) if return_state else None
        ws = _tc_ws(B, T, H, r.device)
        call("rwkv_wkv7_tc_forward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(s0), ptr(y), ptr(cs),
             ptr(s_final), ptr(ws), i32(B), i32(T), i32(H), stream())
        if need_grad:
            # the chunk-parallel products of the forward (10.5 KB per chunk) serve the reverse scan as they are;
            # keeping them costs memory (5 [tokens, C] bf16 units per layer) and saves a prep pass in backward
            ctx.save_for_backward(r, w, k, v, a, b, cs, *((ws,) if WKV7_KEEP_WORKSPACE else ()))
        ctx.has_state = state is not None
        ctx.out_dtype = out_dtype
        ctx.shape = (B, T, H)
        y = y if out_dtype == BF16 else y.to(out_dtype)
        return y, s_final

    @staticmethod
    def backward(ctx, dy, ds_final):
        r, w, k, v, a, b, cs, *kept = ctx.saved_tensors
        B, T, H = ctx.shape
        dy = _c(dy, BF16)
        ds_T = None if ds_final is None else _c(ds_final, torch.float32)
        grads = [torch.empty_like(r) for _ in range(6)]
        ds0 = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device) if ctx.has_state else None
        dstates = torch.empty_like(cs)
        ws = kept[0] if kept else _tc_ws(B, T, H, r.device)
        call("rwkv_wkv7_tc_backward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(dy), ptr(cs), ptr(ds_T),
             ptr(dstates), ptr(ws), i32(1 if kept else 0), *(ptr(g) for g in grads), ptr(ds0), i32(0), i32(B), i32(T),
             i32(H), stream())
        if ctx.out_dtype != BF16:
            grads = [g.to(ctx.out_dtype) for g in grads]
        return (*grads, ds0, None, None)


# "auto": tensor-core chunked kernels from TC_MIN_T steps up, the step-by-step kernels below (decode, short
# chunks).  "simt" / "tc" force one implementation (A/B measurements and tests).
WKV7_IMPL = "auto"
TC_MIN_T = 32
WKV7_KEEP_WORKSPACE = True    # keep the forward's chunk products for the backward (memory for time)


def wkv7(r, w, k, v, a, b, head_size: int = 64, state: Optional[torch.Tensor] = None, return_state: bool = False):
    if head_size != 64:
        raise ValueError("the sm_100a WKV7 kernels are built for head_size 64")
    if r.shape[-1] % 64:
        raise ValueError("channel count must be a multiple of 64")
    use_tc = WKV7_IMPL == "tc" or (WKV7_IMPL == "auto" and r.shape[1] >= TC_MIN_T)
    fn = _WKV7TC if use_tc else _WKV7
    y, s = fn.apply(r, w, k, v, a, b, state, return_state, torch.is_grad_enabled())
    return y, s


# =============================================================================== helpers
def _strip_for(rows_per_batch: int, batch: int, target_ctas: int = 592) -> int:
    """Time steps per CTA: enough CTAs to fill 148 SMs several times, at least 4 steps each."""
    total = rows_per_batch * batch
    strip = max(4, min(64, -(-total // target_ctas)))
    return (strip + 3) // 4 * 4


_PARAM_EPOCH = 0
_F32_CACHE = {}


def bump_param_epoch() -> None:
    """Called after parameters were rewritten behind autograd's back (the optimiser kernels write through raw
    pointers): cached fp32 copies of small parameters are refreshed on next use."""
    global _PARAM_EPOCH
    _PARAM_EPOCH += 1


def _refresh_f32_cache() -> None:
    """Bring every cached fp32 copy up to date with ONE multi-tensor copy (after an optimiser step all of them are
    stale at once: some five hundred 2048-element parameters in a 24-block model, a launch each if done one by one)."""
    dsts, srcs, keys = [], [], []
    for key, (stamp, out, ref_) in list(_F32_CACHE.items()):
        p = ref_()
        if p is None:
            del _F32_CACHE[key]
            continue
        if stamp != (_PARAM_EPOCH, p._version) and p.data_ptr() == key[0]:
            dsts.append(out)
            srcs.append(p.detach().reshape(-1))
            keys.append((key, p))
    if dsts:
        torch._foreach_copy_(dsts, srcs)
        for (key, p), out in zip(keys, dsts):
            _F32_CACHE[key] = ((_PARAM_EPOCH, p._version), out, _F32_CACHE[key][2])


def _f32(t: torch.Tensor) -> torch.Tensor:
    """Flat fp32 copy of a small per-channel parameter.  Copies of ``nn.Parameter`` objects are cached (same
    storage for the life of the parameter, refreshed in place after each optimiser step), which removes a
    dozen tiny conversion kernels per layer and keeps addresses stable for CUDA-graph replay."""
    if not isinstance(t, torch.nn.Parameter):
        return _c(t.detach().reshape(-1), torch.float32)
    key = (t.data_ptr(), t.numel(), t.dtype)
    stamp = (_PARAM_EPOCH, t._version)
    hit = _F32_CACHE.get(key)
    if hit is not None and hit[0] == stamp:
        return hit[1]
    if hit is not None:
        if hit[0][0] != _PARAM_EPOCH and not (t.is_cuda and torch.cuda.is_current_stream_capturing()):
            _refresh_f32_cache()          # an optimiser step has passed: refresh all copies together
            hit = _F32_CACHE.get(key)
            if hit is not None and hit[0] == stamp:
                return hit[1]
        if hit is not None:
            hit[1].copy_(t.detach().reshape(-1))
            _F32_CACHE[key] = (stamp, hit[1], hit[2])
            return hit[1]
    out = t.detach().reshape(-1).float().contiguous()
    _F32_CACHE[key] = (stamp, out, weakref.ref(t))
    return out


def _colsum(partials: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``partials.sum(0)`` for the fp32 per-CTA partial sums ``[n_cta, ...]`` of a backward kernel, delivered in the
    parameters' ``dtype``: one small kernel with coalesced column reads (the framework's reduction takes 28 us for
    592 x 6144 and each bf16 parameter gradient then needs a conversion launch of its own)."""
    if not (partials.is_cuda and partials.dtype == torch.float32 and partials.is_contiguous()
            and dtype in (torch.float32, BF16) and hasattr(_ext.lib(), "rwkv_colsum_f32")):
        return partials.sum(0).to(dtype)
    out = torch.empty(partials.shape[1:], dtype=dtype, device=partials.device)
    call("rwkv_colsum_f32", ptr(partials), i32(partials.shape[0]), i64(out.numel()), ptr(out), i32(1 if dtype == BF16 else 0),
         stream())
    return out


def _param_grad(partials: torch.Tensor, index: int, like: torch.Tensor) -> torch.Tensor:
    return partials[:, index].sum(0).reshape(like.shape).to(like.dtype)


# =============================================================================== LayerNorm / shift / mix
class _LnShiftMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ln_w, ln_b, mix, prev, eps):
        B, T, C = x.shape
        K = mix.numel() // C
        xb = _c(x, BF16)
        w32, b32, m32 = _f32(ln_w), _f32(ln_b), _f32(mix).reshape(K, C)
        pv = None if prev is None else _c(prev, BF16)
        outs = torch.empty(K, B, T, C, dtype=BF16, device=x.device)
        last = torch.empty(B, C, dtype=BF16, device=x.device)
        mean = torch.empty(B * T, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        strip = _strip_for(T, B)
        call("rwkv_ln_shift_mix_forward", ptr(xb), ptr(w32), ptr(b32), ptr(m32), ptr(pv), ptr(outs), ptr(last),
             ptr(mean), ptr(rstd), i32(K), i32(B), i32(T), i32(C), i32(strip), f32(eps), stream())
        ctx.save_for_backward(xb, mean, rstd, w32, b32, m32, pv)
        ctx.meta = (B, T, C, K, strip, x.dtype, ln_w, ln_b, mix, prev is not None)
        if x.dtype != BF16:
            outs, last = outs.to(x.dtype), last.to(x.dtype)
        return outs, last

    @staticmethod
    def backward(ctx, d_outs, d_last):
        return _ln_shift_mix_backward(ctx, list(_c(d_outs, BF16).unbind(0)), d_last)


def _ln_shift_mix_backward(ctx, d_list, d_last, d_res=None):
    """``d_list``: K contiguous bf16 ``[B, T, C]`` gradients (separate allocations are fine: the kernel takes K
    pointers); ``d_res``: gradient of the residual connection around the operator, summed into ``dx`` by the kernel."""
    import ctypes

    xb, mean, rstd, w32, b32, m32, pv = ctx.saved_tensors
    B, T, C, K, strip, xdt, ln_w, ln_b, mix, has_prev = ctx.meta
    dl = None if d_last is None else _c(d_last, BF16)
    dx = torch.empty(B, T, C, dtype=BF16, device=xb.device)
    dprev = torch.empty(B, C, dtype=torch.float32, device=xb.device) if has_prev else None
    n_cta = B * (-(-T // strip))
    partials = torch.empty(n_cta, K + 2, C, dtype=torch.float32, device=xb.device)
    dptrs = (ctypes.c_void_p * K)(*[t.data_ptr() for t in d_list])
    dr = None if d_res is None else _c(d_res, BF16)
    call("rwkv_ln_shift_mix_backward", dptrs, ptr(dl), ptr(dr), ptr(xb), ptr(mean), ptr(rstd), ptr(w32), ptr(b32),
         ptr(m32), ptr(pv), ptr(dx), ptr(dprev), ptr(partials), i32(K), i32(B), i32(T), i32(C), i32(strip),
         stream())
    sums = _colsum(partials, mix.dtype if mix.dtype == ln_w.dtype == ln_b.dtype else torch.float32)
    dmix = sums[:K].reshape(mix.shape).to(mix.dtype)
    dw = sums[K].reshape(ln_w.shape).to(ln_w.dtype)
    db = sums[K + 1].reshape(ln_b.shape).to(ln_b.dtype)
    return dx.to(xdt), dw, db, dmix, (dprev.to(xdt) if has_prev else None), None


class _LnShiftMixUnbound(torch.autograd.Function):
    """Same operator with the K mixed outputs returned as K tensors: their gradients then reach the backward
    kernel as K pointers and are never stacked into one buffer."""

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, mix, prev, eps):
        outs, last = _LnShiftMix.forward(ctx, x, ln_w, ln_b, mix, prev, eps)
        # x is handed back as an output: a residual connection that uses this copy routes its gradient through
        # this node, where the kernel adds it to dx instead of a separate accumulation pass
        return (*outs.unbind(0), last, x.view_as(x))

    @staticmethod
    def backward(ctx, *grads):
        *d_outs, d_last, d_res = grads
        B, T, C = ctx.meta[0], ctx.meta[1], ctx.meta[2]
        zero = None
        d_list = []
        for g in d_outs:
            if g is None:
                if zero is None:
                    zero = torch.zeros(B, T, C, dtype=BF16, device=ctx.saved_tensors[0].device)
                g = zero
            d_list.append(_c(g, BF16))
        return _ln_shift_mix_backward(ctx, d_list, d_last, d_res)


def ln_shift_mix_unbound(x, ln_w, ln_b, mix, prev=None, eps: float = ref.LAYERNORM_EPS):
    """Returns ``((out_0, ..., out_{K-1}), last_row, x)``; use the returned ``x`` for the residual connection."""
    K = mix.numel() // x.shape[-1]
    if K not in (1, 6) or x.shape[-1] % 64:
        outs, last = ref.ln_shift_mix(x, ln_w, ln_b, mix.reshape(K, -1), prev, eps)
        return outs.unbind(0), last, x
    res = _LnShiftMixUnbound.apply(x, ln_w, ln_b, mix, prev, eps)
    return res[:-2], res[-2], res[-1]


def ln_shift_mix(x, ln_w, ln_b, mix, prev=None, eps: float = ref.LAYERNORM_EPS):
    K = mix.numel() // x.shape[-1]
    if K not in (1, 6) or x.shape[-1] % 64:
        return ref.ln_shift_mix(x, ln_w, ln_b, mix.reshape(K, -1), prev, eps)
    return _LnShiftMix.apply(x, ln_w, ln_b, mix, prev, eps)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        C = x.shape[-1]
        xb = _c(x, BF16).reshape(-1, C)
        rows = xb.shape[0]
        w32, b32 = _f32(w), _f32(b)
        y = torch.empty_like(xb)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        strip = _strip_for(rows, 1)
        call("rwkv_layer_norm_forward", ptr(xb), ptr(w32), ptr(b32), ptr(y), ptr(mean), ptr(rstd), i32(rows), i32(C),
             i32(strip), f32(eps), stream())
        ctx.save_for_backward(xb, mean, rstd, w32)
        ctx.meta = (x.shape, x.dtype, strip, w, b)
        return y.reshape(x.shape).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        xb, mean, rstd, w32 = ctx.saved_tensors
        shape, xdt, strip, w, b = ctx.meta
        rows, C = xb.shape
        dyb = _c(dy, BF16).reshape(rows, C)
        dx = torch.empty_like(xb)
        partials = torch.empty(-(-rows // strip), 2, C, dtype=torch.float32, device=xb.device)
        call("rwkv_layer_norm_backward", ptr(dyb), ptr(xb), ptr(mean), ptr(rstd), ptr(w32), ptr(dx), ptr(partials),
             i32(rows), i32(C), i32(strip), stream())
        sums = _colsum(partials, w.dtype if w.dtype == b.dtype else torch.float32)
        return dx.reshape(shape).to(xdt), sums[0].reshape(w.shape).to(w.dtype), sums[1].reshape(b.shape).to(b.dtype), None


def layer_norm(x, weight, bias, eps: float = ref.LAYERNORM_EPS):
    if x.shape[-1] % 8:
        return ref.layer_norm(x, weight, bias, eps)
    return _LayerNorm.apply(x, weight, bias, eps)


# =============================================================================== time-mix prep / post
class _TimemixPrep(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a):
        B, T, C = k.shape
        dt = k.dtype
        layer0 = v_first is None
        kb, vb, wl, al = (_c(t, BF16) for t in (k, v, w_lin, a_lin))
        vf = None if layer0 else _c(v_first, BF16)
        vl = None if layer0 else _c(v_lin, BF16)
        p = [_f32(w0), _f32(a0), None if layer0 else _f32(v0), _f32(k_k), _f32(k_a)]
        outs = [torch.empty(B, T, C, dtype=BF16, device=k.device) for _ in range(5)]
        w_o, k_o, v_o, an_o, b_o = outs
        strip = _strip_for(T, B)
        call("rwkv_timemix_prep_forward", ptr(kb), ptr(vb), ptr(vf), ptr(wl), ptr(al), ptr(vl), *(ptr(t) for t in p),
             ptr(w_o), ptr(k_o), ptr(v_o), ptr(an_o), ptr(b_o), i32(B), i32(T), i32(C), i32(strip), stream())
        if layer0:
            v_o = vb
        ctx.save_for_backward(kb, vb, vf, wl, al, vl, *p)
        ctx.meta = (B, T, C, strip, dt, layer0, [t.shape for t in (w0, a0, k_k, k_a)], [t.dtype for t in (w0, a0, k_k, k_a)])
        res = (w_o, k_o, v_o, an_o, b_o)
        return tuple(t.to(dt) for t in res) if dt != BF16 else res

    @staticmethod
    def backward(ctx, gw, gk, gv, gan, gb):
        kb, vb, vf, wl, al, vl, w0, a0, v0, k_k, k_a = ctx.saved_tensors
        B, T, C, strip, dt, layer0, pshapes, pdtypes = ctx.meta
        dev = kb.device
        zero = None

        def g_(t):
            nonlocal zero
            if t is None:
                if zero is None:
                    zero = torch.zeros(B, T, C, dtype=BF16, device=dev)
                return zero
            return _c(t, BF16)

        gw, gk, gv, gan, gb = (g_(t) for t in (gw, gk, gv, gan, gb))
        dk, dv, dwl, dal = (torch.empty(B, T, C, dtype=BF16, device=dev) for _ in range(4))
        dvf = None if layer0 else torch.empty(B, T, C, dtype=BF16, device=dev)
        dvl = None if layer0 else torch.empty(B, T, C, dtype=BF16, device=dev)
        n_cta = B * (-(-T // strip))
        partials = torch.empty(n_cta, 5, C, dtype=torch.float32, device=dev)
        call("rwkv_timemix_prep_backward", ptr(gw), ptr(gk), ptr(gv), ptr(gan), ptr(gb), ptr(kb), ptr(vb), ptr(vf),
             ptr(wl), ptr(al), ptr(vl), ptr(w0), ptr(a0), ptr(v0), ptr(k_k), ptr(k_a), ptr(dk), ptr(dv), ptr(dvf),
             ptr(dwl), ptr(dal), ptr(dvl), ptr(partials), i32(B), i32(T), i32(C), i32(strip), stream())
        s = _colsum(partials, pdtypes[0] if len(set(pdtypes)) == 1 else torch.float32)
        cast = (lambda t: t.to(dt)) if dt != BF16 else (lambda t: t)
        dw0 = s[0].reshape(pshapes[0]).to(pdtypes[0])
        da0 = s[1].reshape(pshapes[1]).to(pdtypes[1])
        dv0 = None if layer0 else s[2].reshape(pshapes[0]).to(pdtypes[0])
        dkk = s[3].reshape(pshapes[2]).to(pdtypes[2])
        dka = s[4].reshape(pshapes[3]).to(pdtypes[3])
        return (cast(dk), cast(dv), None if layer0 else cast(dvf), cast(dwl), cast(dal),
                None if layer0 else cast(dvl), dw0, da0, dv0, dkk, dka)


def timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, head_size: int = 64):
    if head_size != 64 or k.shape[-1] % 64:
        return ref.timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, head_size)
    return _TimemixPrep.apply(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a)


class _GnBonusGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, r, k, v, g, gn_w, gn_b, r_k, eps):
        B, T, C = y.shape
        dt = y.dtype
        yb, rb, kb, vb, gb_ = (_c(t, BF16) for t in (y, r, k, v, g))
        p = [_f32(gn_w), _f32(gn_b), _f32(r_k)]
        z = torch.empty(B, T, C, dtype=BF16, device=y.device)
        strip = _strip_for(T, B)
        call("rwkv_gn_bonus_gate_forward", ptr(yb), ptr(rb), ptr(kb), ptr(vb), ptr(gb_), *(ptr(t) for t in p), ptr(z),
             i32(B), i32(T), i32(C), i32(strip), f32(eps), stream())
        ctx.save_for_backward(yb, rb, kb, vb, gb_, *p)
        ctx.meta = (B, T, C, strip, dt, eps, (gn_w.shape, gn_b.shape, r_k.shape), (gn_w.dtype, gn_b.dtype, r_k.dtype))
        return z.to(dt)

    @staticmethod
    def backward(ctx, dz):
        yb, rb, kb, vb, gb_, gw, gb, rk = ctx.saved_tensors
        B, T, C, strip, dt, eps, shp, dts = ctx.meta
        dev = yb.device
        dzb = _c(dz, BF16)
        dy, dr, dk, dv, dg = (torch.empty(B, T, C, dtype=BF16, device=dev) for _ in range(5))
        n_cta = B * (-(-T // strip))
        partials = torch.empty(n_cta, 3, C, dtype=torch.float32, device=dev)
        call("rwkv_gn_bonus_gate_backward", ptr(dzb), ptr(yb), ptr(rb), ptr(kb), ptr(vb), ptr(gb_), ptr(gw), ptr(gb),
             ptr(rk), ptr(dy), ptr(dr), ptr(dk), ptr(dv), ptr(dg), ptr(partials), i32(B), i32(T), i32(C), i32(strip),
             f32(eps), stream())
        s = _colsum(partials, dts[0] if len(set(dts)) == 1 else torch.float32)
        cast = (lambda t: t.to(dt)) if dt != BF16 else (lambda t: t)
        return (cast(dy), cast(dr), cast(dk), cast(dv), cast(dg), s[0].reshape(shp[0]).to(dts[0]),
                s[1].reshape(shp[1]).to(dts[1]), s[2].reshape(shp[2]).to(dts[2]), None)


def gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size: int = 64, eps: float = ref.GROUPNORM_EPS):
    if head_size != 64 or y.shape[-1] % 64:
        return ref.gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size, eps)
    return _GnBonusGate.apply(y, r, k, v, g, gn_w, gn_b, r_k, eps)


class _WKV7GN(torch.autograd.Function):
    """Tensor-core WKV7 followed by GroupNorm + bonus + gate as ONE node.  Both halves read ``r``, ``k`` and ``v``;
    as separate nodes autograd sums their two gradients with three extra passes over ``[B, T, C]`` per layer.  Here
    the normalisation backward writes its share first and the WKV7 chunk kernel adds its own in its output pass."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b, g, gn_w, gn_b, r_k, state, return_state: bool, eps: float):
        B, T, C = r.shape
        H = C // 64
        r, w, k, v, a, b, g = (_c(t, BF16) for t in (r, w, k, v, a, b, g))
        s0 = None if state is None else _c(state, torch.float32)
        need_grad = any(ctx.needs_input_grad[:11])
        NC = (T + 15) // 16
        y = torch.empty(B, T, C, dtype=BF16, device=r.device)
        cs = torch.empty(B, H, NC, 64, 64, dtype=BF16, device=r.device) if need_grad else None
        s_final = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device) if return_state else None
        ws = _tc_ws(B, T, H, r.device)
        call("rwkv_wkv7_tc_forward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(s0), ptr(y), ptr(cs),
             ptr(s_final), ptr(ws), i32(B), i32(T), i32(H), stream())
        p = [_f32(gn_w), _f32(gn_b), _f32(r_k)]
        z = torch.empty(B, T, C, dtype=BF16, device=r.device)
        strip = _strip_for(T, B)
        call("rwkv_gn_bonus_gate_forward", ptr(y), ptr(r), ptr(k), ptr(v), ptr(g), *(ptr(t) for t in p), ptr(z),
             i32(B), i32(T), i32(C), i32(strip), f32(eps), stream())
        if need_grad:
            ctx.save_for_backward(r, w, k, v, a, b, g, y, cs, *p, *((ws,) if WKV7_KEEP_WORKSPACE else ()))
        ctx.meta = (B, T, H, strip, eps, state is not None, (gn_w.shape, gn_b.shape, r_k.shape),
                    (gn_w.dtype, gn_b.dtype, r_k.dtype))
        return z, s_final

    @staticmethod
    def backward(ctx, dz, ds_final):
        r, w, k, v, a, b, g, y, cs, gw, gb, rk, *kept = ctx.saved_tensors
        B, T, H, strip, eps, has_state, shp, dts = ctx.meta
        C = H * 64
        dev = r.device
        dzb = _c(dz, BF16)
        dy, dr, dk, dv, dg = (torch.empty(B, T, C, dtype=BF16, device=dev) for _ in range(5))
        n_cta = B * (-(-T // strip))
        partials = torch.empty(n_cta, 3, C, dtype=torch.float32, device=dev)
        call("rwkv_gn_bonus_gate_backward", ptr(dzb), ptr(y), ptr(r), ptr(k), ptr(v), ptr(g), ptr(gw), ptr(gb),
             ptr(rk), ptr(dy), ptr(dr), ptr(dk), ptr(dv), ptr(dg), ptr(partials), i32(B), i32(T), i32(C), i32(strip),
             f32(eps), stream())
        ds_T = None if ds_final is None else _c(ds_final, torch.float32)
        dw, da, db = (torch.empty(B, T, C, dtype=BF16, device=dev) for _ in range(3))
        ds0 = torch.empty(B, H, 64, 64, dtype=torch.float32, device=dev) if has_state else None
        dstates = torch.empty_like(cs)
        ws = kept[0] if kept else _tc_ws(B, T, H, dev)
        call("rwkv_wkv7_tc_backward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(dy), ptr(cs), ptr(ds_T),
             ptr(dstates), ptr(ws), i32(1 if kept else 0), ptr(dr), ptr(dw), ptr(dk), ptr(dv), ptr(da), ptr(db),
             ptr(ds0), i32(1), i32(B), i32(T), i32(H), stream())
        s = _colsum(partials, dts[0] if len(set(dts)) == 1 else torch.float32)
        return (dr, dw, dk, dv, da, db, dg, s[0].reshape(shp[0]).to(dts[0]), s[1].reshape(shp[1]).to(dts[1]),
                s[2].reshape(shp[2]).to(dts[2]), ds0, None, None)


def wkv7_gn(r, w, k, v, a, b, g, gn_w, gn_b, r_k, head_size: int = 64, state=None, return_state: bool = False,
            eps: float = ref.GROUPNORM_EPS):
    """``gn_bonus_gate(wkv7(r, w, k, v, a, b), r, k, v, g, ...)``; returns ``(z, final_state or None)``."""
    use_tc = WKV7_IMPL == "tc" or (WKV7_IMPL == "auto" and r.shape[1] >= TC_MIN_T)
    fusable = (use_tc and head_size == 64 and r.shape[-1] % 64 == 0 and torch.is_grad_enabled()
               and all(t.dtype == BF16 for t in (r, w, k, v, a, b, g)))
    if fusable:
        return _WKV7GN.apply(r, w, k, v, a, b, g, gn_w, gn_b, r_k, state, return_state, eps)
    y, s = wkv7(r, w, k, v, a, b, head_size, state, return_state)
    return gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size, eps), s


class _ReluSq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xb = _c(x, BF16)
        y = torch.empty_like(xb)
        call("rwkv_relu_sq_forward", ptr(xb), ptr(y), i64(xb.numel()), stream())
        ctx.save_for_backward(xb)
        ctx.dt = x.dtype
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        (xb,) = ctx.saved_tensors
        dyb = _c(dy, BF16)
        dx = torch.empty_like(xb)
        call("rwkv_relu_sq_backward", ptr(xb), ptr(dyb), ptr(dx), i64(xb.numel()), i32(0), stream())
        return dx.to(ctx.dt)


def relu_squared(x):
    if x.numel() % 8:
        return ref.relu_squared(x)
    return _ReluSq.apply(x)


# =============================================================================== GEMMs
def linear(x, weight):
    from . import gemm

    return gemm.linear(x, weight)


def matmul(x, w):
    from . import gemm

    return gemm.matmul(x, w)


# =============================================================================== head + loss
class _LinearCrossEntropy(torch.autograd.Function):
    """Vocabulary head, cross-entropy (mean over targets != ignore_index) and L2Wrap without ever
    holding the ``[M, V]`` logits: rows are processed in slabs, and because the loss is a scalar the
    gradients w.r.t. ``x`` and ``weight`` are produced during the forward sweep."""

    SLAB = 4096

    @staticmethod
    def forward(ctx, x, weight, labels, l2wrap, ignore_index, l2wrap_tokens):
        from . import gemm

        M, C = x.shape
        V = weight.shape[0]
        valid = labels != ignore_index
        n_valid = valid.sum().clamp(min=1).float()
        factor = ref.L2WRAP_FACTOR / float(l2wrap_tokens if l2wrap_tokens is not None else M)
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = torch.empty_like(x) if need_x else None
        # bf16 inputs: the weight gradient is accumulated over the slabs in the GEMM epilogue (bf16 [V, C], no fp32
        # temporary of half a gigabyte re-read per slab); other dtypes keep an fp32 accumulator
        dw_in_epilogue = need_w and x.dtype == BF16 and weight.dtype == BF16
        dw = (torch.zeros(V, C, dtype=BF16 if dw_in_epilogue else torch.float32, device=x.device) if need_w else None)
        loss_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        safe_labels = labels.clamp(min=0)
        fused_rows = x.dtype == BF16 and weight.dtype == BF16 and V % 8 == 0
        if fused_rows:
            labels_c = _c(labels, torch.int64)
            inv_n = (1.0 / n_valid).reshape(1)
            loss_rows = torch.empty(M, dtype=torch.float32, device=x.device)
            write_grad = 1 if (need_x or need_w) else 0
        for s in range(0, M, _LinearCrossEntropy.SLAB):
            e = min(M, s + _LinearCrossEntropy.SLAB)
            xs = x[s:e]
            if fused_rows:
                # one statistics sweep + one in-place rewrite of the bf16 slab (logits -> d logits)
                grad = _c(gemm.mm_nt(xs, weight))
                call("rwkv_ce_rows", ptr(grad), ptr(labels_c[s:e]), ptr(inv_n), f32(factor if l2wrap else 0.0),
                     i64(ignore_index), ptr(loss_rows[s:e]), i32(write_grad), i64(e - s), i32(V), stream())
            else:
                logits = gemm.mm_nt(xs, weight).float()
                mx, am = logits.max(dim=-1, keepdim=True)
                ex = torch.exp(logits - mx)
                den = ex.sum(-1, keepdim=True)
                lse = (mx + den.log()).squeeze(-1)
                tgt = logits.gather(-1, safe_labels[s:e, None]).squeeze(-1)
                vs = valid[s:e]
                loss_sum += ((lse - tgt) * vs).sum()
                if need_x or need_w:
                    scale = (vs.float() / n_valid)[:, None]
                    grad = ex / den * scale
                    grad.scatter_add_(-1, safe_labels[s:e, None], -scale)
                    if l2wrap:
                        grad.scatter_add_(-1, am, mx * factor)
                    grad = grad.to(x.dtype)
            if need_x:
                dx[s:e] = gemm.mm_nn(grad, weight)
            if need_w:
                if dw_in_epilogue:
                    gemm.addmm_tn_(dw, grad, xs)
                else:
                    dw += gemm.mm_tn(grad, xs).float()
        if fused_rows:
            loss_sum = loss_rows.sum()
        ctx.save_for_backward(dx, dw)
        ctx.wdtype = weight.dtype
        return loss_sum / n_valid

    @staticmethod
    def backward(ctx, g):
        dx, dw = ctx.saved_tensors
        return (None if dx is None else dx * g.to(dx.dtype), None if dw is None else (dw * g).to(ctx.wdtype),
                None, None, None, None)


def linear_cross_entropy(x, weight, labels, l2wrap=True, ignore_index=-100, l2wrap_tokens=None):
    return _LinearCrossEntropy.apply(x, weight, labels, l2wrap, ignore_index, l2wrap_tokens)


def linear_logprob_entropy(x, weight, targets, temperature: float = 1.0, with_entropy: bool = True):
    from . import loss_kernels

    return loss_kernels.linear_logprob_entropy(x, weight, targets, temperature, with_entropy)


class _LinearReluSq(torch.autograd.Function):
    """``relu(x @ W^T)^2`` with the activation applied in the GEMM epilogue.  Only the output is kept:
    the backward recovers ``relu(pre) = sqrt(y)`` instead of re-reading a saved pre-activation."""

    @staticmethod
    def forward(ctx, x, w):
        from . import gemm_native

        x2 = _c(x.reshape(-1, x.shape[-1]), BF16)
        y = gemm_native.mm_nt(x2, w, epilogue=1)
        ctx.save_for_backward(x2, w, y)
        ctx.shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import gemm

        x2, w, y = ctx.saved_tensors
        dyb = _c(dy.reshape(-1, dy.shape[-1]), BF16)
        dpre = torch.empty_like(y)
        call("rwkv_relu_sq_backward", ptr(y), ptr(dyb), ptr(dpre), i64(y.numel()), i32(1), stream())
        dx = gemm.mm_nn(dpre, w).reshape(ctx.shape) if ctx.needs_input_grad[0] else None
        dw = gemm.mm_tn(dpre, x2) if ctx.needs_input_grad[1] else None
        return dx, dw


class _ChannelMixFFN(torch.autograd.Function):
    """``residual + relu(xk Wk^T)^2 Wv^T`` as one node: relu^2 in the epilogue of the key GEMM, the residual sum in the
    epilogue of the value GEMM, and in backward the activation derivative ``2 sqrt(hidden)`` in the epilogue of the
    value projection's dgrad GEMM (``rwkvtune/models/rwkv7/model.py:304-308`` is the unfused statement)."""

    @staticmethod
    def forward(ctx, xk, wk, wv, residual):
        from . import gemm_native

        x2 = _c(xk.reshape(-1, xk.shape[-1]), BF16)
        r2 = _c(residual.reshape(-1, residual.shape[-1]), BF16)
        hidden = gemm_native.mm_nt(x2, wk, epilogue=1)
        out = gemm_native.mm_nt(hidden, wv, residual=r2)
        ctx.save_for_backward(x2, wk, wv, hidden)
        ctx.shape = xk.shape
        return out.reshape(residual.shape)

    @staticmethod
    def backward(ctx, dout):
        from . import gemm, gemm_native

        x2, wk, wv, hidden = ctx.saved_tensors
        d2 = _c(dout.reshape(-1, dout.shape[-1]), BF16)
        dpre = gemm_native.mm_nn(d2, wv, epilogue=5, residual=hidden)        # (dout Wv) * 2 sqrt(hidden)
        dwv = gemm.mm_tn(d2, hidden) if ctx.needs_input_grad[2] else None
        dx = gemm.mm_nn(dpre, wk).reshape(ctx.shape) if ctx.needs_input_grad[0] else None
        dwk = gemm.mm_tn(dpre, x2) if ctx.needs_input_grad[1] else None
        return dx, dwk, dwv, (dout if ctx.needs_input_grad[3] else None)


def channel_mix_ffn(xk, wk, wv, residual):
    from . import gemm_native

    x2 = xk.reshape(-1, xk.shape[-1])
    r2 = residual.reshape(-1, residual.shape[-1])
    ok = (xk.dtype == BF16 and wk.dtype == BF16 and wv.dtype == BF16 and residual.dtype == BF16
          and x2.is_contiguous() and r2.is_contiguous() and gemm_native.native_ok(x2, wk, "nt")
          and x2.shape[0] >= gemm_native.MIN_M and wk.shape[0] % 8 == 0 and wv.shape[0] % 8 == 0)
    if ok:   # the value projection contracts over 4C: without split-K it needs enough output tiles of its own
        tiles = -(-x2.shape[0] // 128) * -(-wv.shape[0] // 256)
        ok = tiles >= 64 or wv.shape[1] <= 4096
    if ok:
        return _ChannelMixFFN.apply(xk, wk, wv, residual)
    from . import gemm

    return gemm.linear_add(linear_relu_sq(xk, wk), wv, residual)


def linear_relu_sq(x, weight):
    from . import gemm_native

    x2 = x.reshape(-1, x.shape[-1])
    if not torch.is_grad_enabled():
        from . import gemm

        ys = gemm.decode_products([x], [weight], acts=["relu_sq"])
        if ys is not None:
            return ys[0]
    if x.dtype == BF16 and weight.dtype == BF16 and gemm_native.native_ok(x2 if x2.is_contiguous() else x2.contiguous(), weight, "nt"):
        return _LinearReluSq.apply(x, weight)
    return relu_squared(linear(x, weight))


# =============================================================================== WKV7, chunked tensor-core form
def wkv7_tc_forward(r, w, k, v, a, b, state=None, return_state=False, save_chunk_states=False):
    """Forward only (no autograd): returns ``(y, final_state or None, chunk_start_states or None)``."""
    B, T, C = r.shape
    H = C // 64
    r, w, k, v, a, b = (_c(t, BF16) for t in (r, w, k, v, a, b))
    s0 = None if state is None else _c(state, torch.float32)
    y = torch.empty(B, T, C, dtype=BF16, device=r.device)
    NC = (T + 15) // 16
    cs = torch.empty(B, H, NC, 64, 64, dtype=BF16, device=r.device) if save_chunk_states else None
    sf = torch.empty(B, H, 64, 64, dtype=torch.float32, device=r.device) if return_state else None
    ws = _tc_ws(B, T, H, r.device)
    call("rwkv_wkv7_tc_forward", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(s0), ptr(y), ptr(cs), ptr(sf),
         ptr(ws), i32(B), i32(T), i32(H), stream())
    return y, sf, cs


def wkv7_pool_step(r, w, k, v, a, b, pool: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """WKV7 forward (no autograd) that updates ``pool[slots[i]]`` (fp32 ``[n_slots, H, 64, 64]``) in place for
    sequence ``i``: decode or prefill of any subset of a state pool without gathering or scattering states."""
    B, T, C = r.shape
    H = C // 64
    if pool.dtype != torch.float32 or not pool.is_contiguous() or tuple(pool.shape[1:]) != (H, 64, 64):
        raise ValueError("pool must be a contiguous fp32 [n_slots, H, 64, 64] tensor")
    r, w, k, v, a, b = (_c(t, BF16) for t in (r, w, k, v, a, b))
    slots = _c(slots, torch.int64)
    y = torch.empty(B, T, C, dtype=BF16, device=r.device)
    call("rwkv_wkv7_forward_slots", ptr(r), ptr(w), ptr(k), ptr(v), ptr(a), ptr(b), ptr(pool), ptr(slots), ptr(y),
         i32(B), i32(T), i32(H), stream())
    return y


def timemix_decode_core_ok(r, g, state, head_size: int) -> bool:
    """One token per sequence, bf16, head size 64, an existing fp32 state (tensor, or ``(pool, slots)``), no autograd,
    and the fused kernel present in the library."""
    if not (r.is_cuda and r.dim() == 3 and r.shape[1] == 1 and r.dtype == BF16 and g.dtype == BF16 and head_size == 64
            and r.shape[-1] % 64 == 0 and 0 < r.shape[0] <= 65535 and not torch.is_grad_enabled() and state is not None):
        return False
    from . import _ext

    if not hasattr(_ext.lib(), "rwkv_wkv7_decode_core"):
        return False
    st = state[0] if isinstance(state, tuple) else state
    return st.dtype == torch.float32 and st.is_contiguous() and tuple(st.shape[1:]) == (r.shape[-1] // 64, 64, 64)


def timemix_decode_core(r, k, v, v_first, w_lin, a_lin, v_lin, g, w0, a0, v0, k_k, k_a, r_k, gn_w, gn_b, state,
                        eps: float = ref.GROUPNORM_EPS):
    """Key/decay/value preparation, WKV7 state update + read-out and GroupNorm + bonus + gate of one decoding step as
    ONE kernel (``csrc/wkv7_decode.cu``); same roundings and summation order as ``timemix_prep`` -> ``wkv7`` ->
    ``gn_bonus_gate``.
    ``state``: fp32 ``[B, H, 64, 64]`` (a new tensor is returned, or the same one while ``INPLACE_STATE``) or
    ``(pool, slots)`` (updated in place).  ``v_first`` / ``v_lin`` are ``None`` in the first block.
    Returns ``(z [B, 1, C] bf16, new state)``."""
    B, _, C = r.shape
    H = C // 64
    r, k, v, w_lin, a_lin, g = (_c(t, BF16) for t in (r, k, v, w_lin, a_lin, g))
    if v_first is not None:
        v_first, v_lin = _c(v_first, BF16), _c(v_lin, BF16)
    slots = None
    if isinstance(state, tuple):
        s_in = s_out = state[0]
        slots = _c(state[1], torch.int64)
        new_state = state
    else:
        s_in = state
        s_out = state if INPLACE_STATE else torch.empty_like(state)
        new_state = s_out
    z = torch.empty(B, 1, C, dtype=BF16, device=r.device)
    call("rwkv_wkv7_decode_core", ptr(r), ptr(k), ptr(v), ptr(w_lin), ptr(a_lin), ptr(v_lin), ptr(v_first), ptr(g),
         ptr(_f32(w0)), ptr(_f32(a0)), ptr(_f32(v0)) if v_first is not None else ptr(None), ptr(_f32(k_k)), ptr(_f32(k_a)),
         ptr(_f32(r_k)), ptr(_f32(gn_w)), ptr(_f32(gn_b)), ptr(s_in), ptr(s_out), ptr(slots), ptr(z), i32(B), i32(H),
         f32(eps), stream())
    return z, new_state


# =============================================================================== gathers
def gather_rows(src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``src.index_select(0, index)`` for a contiguous tensor whose rows are a multiple of 16 bytes."""
    src = _c(src)
    index = _c(index, torch.int64)
    row_bytes = (src.numel() // max(src.shape[0], 1)) * src.element_size()
    if row_bytes % 16 or src.data_ptr() % 16:
        return src.index_select(0, index)
    out = torch.empty((index.numel(),) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    call("rwkv_gather_rows", ptr(src), ptr(index), ptr(out), i64(index.numel()), i64(src.shape[0]), i64(row_bytes),
         stream())
    return out


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight):
        ctx.save_for_backward(idx)
        ctx.wshape = weight.shape
        return gather_rows(weight, idx.reshape(-1)).reshape(*idx.shape, weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        V, C = ctx.wshape
        dyb = _c(dy.reshape(-1, C), BF16)
        sorted_idx, order = torch.sort(idx.reshape(-1).to(torch.int64), stable=True)
        dW = torch.zeros(V, C, dtype=BF16, device=dy.device)
        call("rwkv_embedding_backward", ptr(dyb), ptr(sorted_idx), ptr(order), ptr(dW), i64(dyb.shape[0]), i64(V),
             i32(C), stream())
        return None, dW


def embedding(idx, weight):
    if weight.dtype != BF16 or weight.shape[1] % 8:
        return torch.nn.functional.embedding(idx, weight)
    return _Embedding.apply(idx, weight)
