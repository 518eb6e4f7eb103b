"""Step-by-step WKV7 with a closed-form backward: the second, autograd-free oracle of the chunk-step operator.

Counterpart of ``rwkvtune/models/rwkv7/operators/wkv_infctx_naive.py`` (``naive_recurrent_rwkv7_fwd`` ``:11-70``,
``naive_recurrent_rwkv7_bwd`` ``:73-197``, ``RWKV7InfctxNaiveFunction`` ``:200-225``) and of the autograd wrapper in
``wkv_infctx.py:18-153`` (``WKV7InfctxFunction``).  Tensors are ``[B, T, H, N]``; the state is ``[B, H, N, N]``
indexed ``[value_row, key_col]``; everything is computed in fp32.

Per head and step, with ``d_t = exp(-exp(w_t))`` and ``q_t`` already multiplied by ``scale``::

    u_t = S_{t-1} a_t                      (N values)
    S_t = S_{t-1} diag(d_t) + u_t b_t^T + v_t k_t^T
    y_t = S_t q_t

The backward walks the steps in reverse with ``G`` = dL/dS_t (seeded by the gradient of the final state)::

    G  += dy_t q_t^T            dq_t = S_t^T dy_t
    dv_t = G k_t                dk_t = G^T v_t
    db_t = G^T u_t              e_t  = G b_t            da_t = S_{t-1}^T e_t
    dd_t = colsum(G * S_{t-1})  dw_t = -dd_t d_t exp(w_t)
    G   = G diag(d_t) + e_t a_t^T                       (now dL/dS_{t-1})

The forward keeps every ``S_t`` (T+1 states), which is what makes this an oracle and not a training kernel: the
CUDA kernels keep one state per 16-step chunk and rebuild the rest.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

__all__ = ["naive_recurrent_rwkv7_fwd", "naive_recurrent_rwkv7_bwd", "RWKV7InfctxNaiveFunction", "WKV7InfctxFunction"]


def _f32(*ts):
    return [t.float() for t in ts]


def _states(q, k, v, w, a, b, initial_state) -> Tuple[List[torch.Tensor], torch.Tensor]:
    """All states ``S_0 .. S_T`` (list of ``[B, H, N, N]``) and the decays ``d`` ``[B, T, H, N]``."""
    B, T, H, N = q.shape
    S = (torch.zeros(B, H, N, N, dtype=torch.float32, device=q.device) if initial_state is None
         else initial_state.float())
    d = torch.exp(-torch.exp(w))
    states = [S]
    for t in range(T):
        u = torch.einsum("bhij,bhj->bhi", S, a[:, t])
        S = S * d[:, t, :, None, :] + u[..., None] * b[:, t, :, None, :] + v[:, t, :, :, None] * k[:, t, :, None, :]
        states.append(S)
    return states, d


def naive_recurrent_rwkv7_fwd(q, k, v, w, a, b, scale: float = 1.0, initial_state: Optional[torch.Tensor] = None):
    """``(output [B, T, H, N] fp32, final_state [B, H, N, N] fp32)``; ``w`` is the raw decay input."""
    q, k, v, w, a, b = _f32(q, k, v, w, a, b)
    states, _ = _states(q, k, v, w, a, b, initial_state)
    qs = q * scale
    y = torch.stack([torch.einsum("bhij,bhj->bhi", states[t + 1], qs[:, t]) for t in range(q.shape[1])], dim=1)
    return y, states[-1]


def naive_recurrent_rwkv7_bwd(q, k, v, w, a, b, doutput, dh_t: Optional[torch.Tensor] = None, scale: float = 1.0,
                              initial_state: Optional[torch.Tensor] = None):
    """``(dq, dk, dv, dw, da, db, dh0)`` in fp32 from the output gradient and the gradient of the final state."""
    q, k, v, w, a, b, dy = _f32(q, k, v, w, a, b, doutput)
    B, T, H, N = q.shape
    states, d = _states(q, k, v, w, a, b, initial_state)
    qs = q * scale
    G = torch.zeros(B, H, N, N, dtype=torch.float32, device=q.device) if dh_t is None else dh_t.float().clone()
    dq, dk, dv, dw, da, db = (torch.empty_like(q) for _ in range(6))
    for t in range(T - 1, -1, -1):
        S_prev, S_cur = states[t], states[t + 1]
        G = G + dy[:, t, :, :, None] * qs[:, t, :, None, :]
        dq[:, t] = torch.einsum("bhij,bhi->bhj", S_cur, dy[:, t]) * scale
        dv[:, t] = torch.einsum("bhij,bhj->bhi", G, k[:, t])
        dk[:, t] = torch.einsum("bhij,bhi->bhj", G, v[:, t])
        u = torch.einsum("bhij,bhj->bhi", S_prev, a[:, t])
        db[:, t] = torch.einsum("bhij,bhi->bhj", G, u)
        e = torch.einsum("bhij,bhj->bhi", G, b[:, t])
        da[:, t] = torch.einsum("bhij,bhi->bhj", S_prev, e)
        dd = (G * S_prev).sum(dim=2)
        dw[:, t] = -dd * d[:, t] * torch.exp(w[:, t])
        G = G * d[:, t, :, None, :] + e[..., None] * a[:, t, :, None, :]
    return dq, dk, dv, dw, da, db, G


class RWKV7InfctxNaiveFunction(torch.autograd.Function):
    """``apply(q, k, v, w, a, b, scale, initial_state) -> (output, final_state)`` with the closed-form backward."""

    @staticmethod
    def forward(ctx, q, k, v, w, a, b, scale, initial_state):
        y, final = naive_recurrent_rwkv7_fwd(q, k, v, w, a, b, scale, initial_state)
        ctx.save_for_backward(q, k, v, w, a, b, *(() if initial_state is None else (initial_state,)))
        ctx.scale = scale
        return y, final

    @staticmethod
    def backward(ctx, dy, dfinal):
        q, k, v, w, a, b, *rest = ctx.saved_tensors
        s0 = rest[0] if rest else None
        grads = naive_recurrent_rwkv7_bwd(q, k, v, w, a, b, dy, dfinal, ctx.scale, s0)
        cast = [g.to(t.dtype) for g, t in zip(grads[:6], (q, k, v, w, a, b))]
        return (*cast, None, grads[6] if s0 is not None else None)


class WKV7InfctxFunction(torch.autograd.Function):
    """``apply(w, q, k, v, a, b, state) -> (output, final_state)``: the chunk step on this package's kernels (CUDA
    tensors) or on the fp32 recurrence (CPU tensors), wrapped so that code which calls the reference's autograd
    class directly keeps working.  Gradients flow to the six inputs and to ``state``."""

    @staticmethod
    def forward(ctx, w, q, k, v, a, b, state):
        from . import rwkv7_wkv_infctx

        with torch.enable_grad():
            leaves = [t.detach().requires_grad_(True) for t in (w, q, k, v, a, b)]
            s0 = state.detach().requires_grad_(True)
            y, s1 = rwkv7_wkv_infctx(*leaves, s0)
        ctx.graph = (leaves, s0, y, s1)
        return y.detach(), s1.detach()

    @staticmethod
    def backward(ctx, dy, ds):
        leaves, s0, y, s1 = ctx.graph
        ctx.graph = None
        grads = torch.autograd.grad([y, s1], leaves + [s0], [dy, torch.zeros_like(s1) if ds is None else ds],
                                    allow_unused=True)
        return tuple(grads)
