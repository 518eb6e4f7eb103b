"""Host-CPU implementations that are faster than letting autograd trace the plain statements.

``wkv7`` is the recurrence of :func:`rwkvtune_b200.ops.reference.wkv7` as one autograd node: the forward keeps every
state ``S_0 .. S_T`` in one buffer, the backward is the closed-form reverse recurrence (the algebra is spelled out in
``models/rwkv7/operators/infctx_oracle.py``).  Everything that does not depend on the running state is batched over
time (the outer products ``v k^T``, the read-out ``S_t r_t``, ``u_t = S_{t-1} a_t``, the gradients of ``r`` and ``a``);
what is left in the Python loops is three small batched operations per step forward and seven backward, against the
several dozen that autograd records for the traced statement (each ``x[:, t]`` alone costs a full-size zero fill in
its backward).  On the 0.1B model at 2 x 256 tokens that takes a CPU training step from 6.8 s to 3.0 s; the reference's
CPU operator (``rwkvtune/models/rwkv7/operators/wkv_cpu.py:9-80``, traced by autograd) needs 5.9 s on the same
machine.  When the native library is built the same algebra runs there (``csrc/wkv7_cpu.cpp``: one (batch, head)
problem per thread, vectorised rows, one kept state per 16 steps and the rest rebuilt in the backward), which brings
the step to 2.1 s; the PyTorch form remains the fallback, and the traced statement stays the oracle of the tests.
``RWKVTUNE_NATIVE_CPU=0`` keeps everything in PyTorch.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

_NATIVE = None
_NATIVE_TRIED = False


def _native_lib():
    """The package's native library when it carries the host WKV7 functions (``csrc/wkv7_cpu.cpp``); ``None`` when it
    is not built or ``RWKVTUNE_NATIVE_CPU=0``.  The pure-PyTorch forms below are the fallback."""
    global _NATIVE, _NATIVE_TRIED
    if not _NATIVE_TRIED:
        _NATIVE_TRIED = True
        if os.environ.get("RWKVTUNE_NATIVE_CPU", "1") != "0":
            path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "librwkvtune_b200.so")
            try:
                lib = ctypes.CDLL(path)
                lib.rwkv_wkv7_cpu_forward.argtypes = [ctypes.c_void_p] * 11 + [ctypes.c_int] * 5
                lib.rwkv_wkv7_cpu_backward.argtypes = [ctypes.c_void_p] * 17 + [ctypes.c_int] * 5
                lib.rwkv_wkv7_cpu_history_states.argtypes = [ctypes.c_int]
                _NATIVE = lib
            except (OSError, AttributeError):
                _NATIVE = None
    return _NATIVE


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _threads(work_items: int) -> int:
    return max(1, min(torch.get_num_threads(), work_items))


def _flat32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().float().contiguous()


class _WKV7Native(torch.autograd.Function):
    """The recurrence in the native library: one (batch, head) problem per thread, state history kept for the backward."""

    @staticmethod
    def forward(ctx, r, w, k, v, a, b, state, head_size: int):
        lib = _native_lib()
        B, T, C = r.shape
        N = head_size
        H = C // N
        ins = [_flat32(t) for t in (r, w, k, v, a, b)]
        s0 = None if state is None else _flat32(state)
        history = torch.empty(B * H, lib.rwkv_wkv7_cpu_history_states(T), N, N, dtype=torch.float32)
        decay = torch.empty(B, T, C, dtype=torch.float32)
        y = torch.empty(B, T, C, dtype=torch.float32)
        final = torch.empty(B, H, N, N, dtype=torch.float32)
        rc = lib.rwkv_wkv7_cpu_forward(*[_p(t) for t in ins], _p(s0), _p(history), _p(final), _p(y), _p(decay), B, T, H, N,
                                       _threads(B * H))
        if rc != 0:
            raise RuntimeError(f"rwkv_wkv7_cpu_forward refused the shapes (status {rc})")
        ctx.save_for_backward(*ins, decay, history)
        ctx.dims = (B, T, H, N)
        ctx.dtypes = tuple(t.dtype for t in (r, w, k, v, a, b))
        ctx.state_dtype = None if state is None else state.dtype
        return y, final

    @staticmethod
    def backward(ctx, dy, dstate):
        lib = _native_lib()
        r, w, k, v, a, b, decay, history = ctx.saved_tensors
        B, T, H, N = ctx.dims
        dy = _flat32(dy)
        ds = None if dstate is None else _flat32(dstate)
        grads = [torch.empty(B, T, H * N, dtype=torch.float32) for _ in range(6)]
        ds0 = torch.empty(B, H, N, N, dtype=torch.float32) if ctx.state_dtype is not None else None
        rc = lib.rwkv_wkv7_cpu_backward(_p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(decay), _p(history), _p(dy), _p(ds),
                                        *[_p(g) for g in grads], _p(ds0), B, T, H, N, _threads(B * H))
        if rc != 0:
            raise RuntimeError(f"rwkv_wkv7_cpu_backward refused the shapes (status {rc})")
        out = [g.to(dt) for g, dt in zip(grads, ctx.dtypes)]
        return (*out, None if ds0 is None else ds0.to(ctx.state_dtype), None)


def _wkv7_native_nograd(r, w, k, v, a, b, head_size: int, state):
    lib = _native_lib()
    B, T, C = r.shape
    N = head_size
    H = C // N
    ins = [_flat32(t) for t in (r, w, k, v, a, b)]
    s0 = None if state is None else _flat32(state)
    y = torch.empty(B, T, C, dtype=torch.float32)
    final = torch.empty(B, H, N, N, dtype=torch.float32)
    rc = lib.rwkv_wkv7_cpu_forward(*[_p(t) for t in ins], _p(s0), None, _p(final), _p(y), None, B, T, H, N, _threads(B * H))
    if rc != 0:
        raise RuntimeError(f"rwkv_wkv7_cpu_forward refused the shapes (status {rc})")
    return y, final


def _time_major(t: torch.Tensor, B: int, T: int, H: int, N: int) -> torch.Tensor:
    """``[B, T, H*N]`` (any float dtype) -> contiguous fp32 ``[T, B*H, N]``."""
    return t.float().reshape(B, T, H, N).permute(1, 0, 2, 3).reshape(T, B * H, N).contiguous()


def _batch_major(t: torch.Tensor, B: int, T: int, H: int, N: int) -> torch.Tensor:
    return t.reshape(T, B, H, N).permute(1, 0, 2, 3).reshape(B, T, H * N)


def _run_states(w, k, v, a, b, state0: Optional[torch.Tensor], BH: int, T: int, N: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """All states ``[T+1, BH, N, N]`` (index ``[value_row, key_col]``) and the decays ``d = exp(-exp(w))``."""
    d = torch.exp(-torch.exp(w))
    states = torch.empty(T + 1, BH, N, N, dtype=torch.float32, device=w.device)
    if state0 is None:
        states[0].zero_()
    else:
        states[0].copy_(state0.reshape(BH, N, N))
    # S_t starts as v_t k_t^T for every t at once; the loop adds the two terms that depend on S_{t-1}
    torch.mul(v.unsqueeze(-1), k.unsqueeze(-2), out=states[1:])
    a_col = a.unsqueeze(-1)
    b_row = b.unsqueeze(-2)
    d_row = d.unsqueeze(-2)
    for t in range(T):
        prev, cur = states[t], states[t + 1]
        u = torch.bmm(prev, a_col[t])                     # [BH, N, 1]
        cur.addcmul_(prev, d_row[t])
        cur.baddbmm_(u, b_row[t])
    return states, d


class _WKV7(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, w, k, v, a, b, state, head_size: int):
        B, T, C = r.shape
        N = head_size
        H = C // N
        BH = B * H
        tm = [_time_major(t, B, T, H, N) for t in (r, w, k, v, a, b)]
        states, d = _run_states(tm[1], tm[2], tm[3], tm[4], tm[5], state, BH, T, N)
        y = torch.bmm(states[1:].reshape(T * BH, N, N), tm[0].reshape(T * BH, N, 1)).reshape(T, BH, N)
        ctx.save_for_backward(*tm, d, states)
        ctx.shape = (B, T, H, N)
        ctx.dtypes = tuple(t.dtype for t in (r, w, k, v, a, b))
        ctx.state_dtype = None if state is None else state.dtype
        return _batch_major(y, B, T, H, N), states[T].reshape(B, H, N, N).clone()

    @staticmethod
    def backward(ctx, dy, dstate):
        r, w, k, v, a, b, d, states = ctx.saved_tensors
        B, T, H, N = ctx.shape
        BH = B * H
        dy = _time_major(dy, B, T, H, N)
        G = (torch.zeros(BH, N, N, dtype=torch.float32, device=dy.device) if dstate is None
             else dstate.float().reshape(BH, N, N).clone())
        prev_all = states[:-1].reshape(T * BH, N, N)
        u = torch.bmm(prev_all, a.reshape(T * BH, N, 1)).reshape(T, BH, N)            # u_t = S_{t-1} a_t
        kb = torch.stack([k, b], dim=-1)                                                # [T, BH, N, 2]
        vu = torch.stack([v, u], dim=-2)                                                # [T, BH, 2, N]
        right = torch.empty(T, BH, N, 2, dtype=torch.float32, device=dy.device)         # G k  |  G b
        left = torch.empty(T, BH, 2, N, dtype=torch.float32, device=dy.device)          # G^T v  |  G^T u
        dd = torch.empty(T, BH, N, dtype=torch.float32, device=dy.device)
        dy_col, r_row = dy.unsqueeze(-1), r.unsqueeze(-2)
        a_row, d_row = a.unsqueeze(-2), d.unsqueeze(-2)
        scratch = torch.empty(BH, N, N, dtype=torch.float32, device=dy.device)
        for t in range(T - 1, -1, -1):
            G.baddbmm_(dy_col[t], r_row[t])                                             # now dL/dS_t
            torch.bmm(G, kb[t], out=right[t])
            torch.bmm(vu[t], G, out=left[t])
            torch.mul(G, states[t], out=scratch)
            torch.sum(scratch, dim=1, out=dd[t])
            G.mul_(d_row[t])
            G.baddbmm_(right[t, :, :, 1:], a_row[t])                                    # now dL/dS_{t-1}
        dv, e = right[..., 0], right[..., 1]
        dk, db = left[:, :, 0], left[:, :, 1]
        dr = torch.bmm(dy.reshape(T * BH, 1, N), states[1:].reshape(T * BH, N, N)).reshape(T, BH, N)
        da = torch.bmm(e.reshape(T * BH, 1, N), prev_all).reshape(T, BH, N)
        dw = -dd * d * torch.exp(w)
        grads = [_batch_major(g, B, T, H, N).to(dt) for g, dt in zip((dr, dw, dk, dv, da, db), ctx.dtypes)]
        dstate0 = None if ctx.state_dtype is None else G.reshape(B, H, N, N).to(ctx.state_dtype)
        return (*grads, dstate0, None)


def wkv7(r, w, k, v, a, b, head_size: int = 64, state: Optional[torch.Tensor] = None):
    """Same contract as :func:`rwkvtune_b200.ops.reference.wkv7`: ``[B, T, C]`` inputs, optional state
    ``[B, H, N, N]``; returns ``(y [B, T, C] fp32, final_state [B, H, N, N] fp32)``.  With autograd off nothing but
    the running state is kept."""
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (r, w, k, v, a, b, state))
    native = r.device.type == "cpu" and head_size <= 256 and r.shape[1] > 0 and _native_lib() is not None
    if needs_grad:
        return (_WKV7Native if native else _WKV7).apply(r, w, k, v, a, b, state, head_size)
    if native:
        return _wkv7_native_nograd(r, w, k, v, a, b, head_size, state)
    B, T, C = r.shape
    N = head_size
    H = C // N
    BH = B * H
    rt, wt, kt, vt, at, bt = (_time_major(t, B, T, H, N) for t in (r, w, k, v, a, b))
    d = torch.exp(-torch.exp(wt))
    S = (torch.zeros(BH, N, N, dtype=torch.float32, device=r.device) if state is None
         else state.float().reshape(BH, N, N).clone())
    y = torch.empty(T, BH, N, dtype=torch.float32, device=r.device)
    for t in range(T):
        u = torch.bmm(S, at[t].unsqueeze(-1))
        S.mul_(d[t].unsqueeze(-2))
        S.baddbmm_(u, bt[t].unsqueeze(-2))
        S.baddbmm_(vt[t].unsqueeze(-1), kt[t].unsqueeze(-2))
        torch.bmm(S, rt[t].unsqueeze(-1), out=y[t].unsqueeze(-1))
    return _batch_major(y, B, T, H, N), S.reshape(B, H, N, N)


def grad_norm_sq(g: torch.Tensor, scale: float) -> torch.Tensor:
    """``sum((g * scale)^2)`` of a flat gradient without the two full-size temporaries of the plain statement (a BLAS
    dot product: 10 ms instead of 190 ms for the 191 M parameters of the 0.1B model)."""
    gf = g if g.dtype == torch.float32 else g.float()
    return torch.dot(gf.reshape(-1), gf.reshape(-1)) * (scale * scale)


def adamw_step(p32, g, m, v, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               grad_scale: float = 1.0, scratch: Optional[torch.Tensor] = None):
    """:func:`rwkvtune_b200.ops.reference.adamw_step` with the gradient scale folded into the moment updates and the
    denominator formed in a caller-kept ``scratch`` buffer, so that a step allocates nothing of parameter size."""
    gf = g if g.dtype == torch.float32 else g.float()
    m.mul_(beta1).add_(gf, alpha=(1 - beta1) * grad_scale)
    v.mul_(beta2).addcmul_(gf, gf, value=(1 - beta2) * grad_scale * grad_scale)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = torch.div(v, bc2, out=scratch) if scratch is not None and scratch.shape == v.shape else v / bc2
    denom.sqrt_().add_(eps)
    p32.mul_(1 - lr * weight_decay).addcdiv_(m, denom, value=-lr / bc1)
    return p32
