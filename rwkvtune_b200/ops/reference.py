"""Plain-PyTorch statements of every fused operator.

These functions are the CPU execution path and the numerical oracle for the
sm_100a kernels: each CUDA kernel in ``rwkvtune_b200/csrc`` is tested against
the function of the same name here evaluated in fp32.  All of them are
differentiable through ordinary autograd.

Math source: ``rwkvtune/models/rwkv7/model.py:134-172`` (time mix),
``:304-308`` (channel mix), ``rwkvtune/models/rwkv7/operators/wkv_cpu.py:61-68``
(WKV7 recurrence), ``rwkvtune/training/lightning_module.py:23-39`` (L2Wrap).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

GROUPNORM_EPS = 64e-5
LAYERNORM_EPS = 1e-5
L2WRAP_FACTOR = 1e-4


# --------------------------------------------------------------------------- WKV7
def wkv7(r, w, k, v, a, b, head_size: int = 64, state: Optional[torch.Tensor] = None):
    """Sequential WKV7 recurrence in fp32.

    Inputs are ``[B, T, C]``; ``state`` is ``[B, H, N, N]`` indexed
    ``[value_row, key_col]``.  Per head and step, with ``d = exp(-exp(w))``::

        sa = S a;  S = S diag(d) + sa b^T + v k^T;  y = S r

    Returns ``(y [B,T,C] fp32, final_state [B,H,N,N] fp32)``.
    """
    B, T, C = r.shape
    N = head_size
    H = C // N
    f = lambda t: t.reshape(B, T, H, N).float()
    r_, k_, v_, a_, b_ = f(r), f(k), f(v), f(a), f(b)
    d_ = torch.exp(-torch.exp(f(w)))
    S = torch.zeros(B, H, N, N, dtype=torch.float32, device=r.device) if state is None else state.float()
    ys = []
    for t in range(T):
        sa = torch.einsum("bhij,bhj->bhi", S, a_[:, t])
        S = S * d_[:, t, :, None, :] + sa[..., :, None] * b_[:, t, :, None, :] + v_[:, t, :, :, None] * k_[:, t, :, None, :]
        ys.append(torch.einsum("bhij,bhj->bhi", S, r_[:, t]))
    y = torch.stack(ys, dim=1).reshape(B, T, C)
    return y, S


# --------------------------------------------------------------------------- norms / shifts
def layer_norm(x, weight, bias, eps: float = LAYERNORM_EPS):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


def token_shift(h: torch.Tensor, prev: Optional[torch.Tensor]) -> torch.Tensor:
    """``h[t-1]`` with zeros (or the carried last row ``prev [B, C]``) at ``t = 0``."""
    first = torch.zeros_like(h[:, :1]) if prev is None else prev.to(h.dtype).unsqueeze(1)
    return torch.cat([first, h[:, :-1]], dim=1)


def ln_shift_mix(x, ln_w, ln_b, mix, prev: Optional[torch.Tensor] = None, eps: float = LAYERNORM_EPS):
    """LayerNorm, token shift and ``K`` lerps in one step.

    ``mix`` is ``[K, C]``.  Returns ``(outs [K, B, T, C], last_row [B, C])`` where
    ``outs[i] = h + (shift(h) - h) * mix[i]`` and ``h = LayerNorm(x)``;
    ``last_row`` is ``h[:, -1]`` (the value carried to the next chunk).
    """
    h = F.layer_norm(x.float(), (x.shape[-1],), ln_w.float(), ln_b.float(), eps)
    delta = token_shift(h, None if prev is None else prev.float()) - h
    mix = mix.reshape(-1, x.shape[-1])
    outs = h.unsqueeze(0) + delta.unsqueeze(0) * mix.float().reshape(mix.shape[0], 1, 1, -1)
    return outs.to(x.dtype), h[:, -1].to(x.dtype)


# --------------------------------------------------------------------------- time-mix pre/post
def timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, head_size: int = 64):
    """Everything between the projections and the WKV7 recurrence.

    ``w = -softplus(-(w0 + w_lin)) - 0.5``; ``a = sigmoid(a0 + a_lin)``;
    ``v <- v + (v_first - v) * sigmoid(v0 + v_lin)`` unless ``v_first is None``
    (layer 0); ``kk = normalize_per_head(k * k_k)``; ``k <- k * (1 + (a-1) * k_a)``.
    Returns ``(w, k_mod, v_mix, -kk, kk * a)`` in the dtype of ``k``.
    """
    dt = k.dtype
    B, T, C = k.shape
    kf, vf = k.float(), v.float()
    w = -F.softplus(-(w0.float().reshape(1, 1, C) + w_lin.float())) - 0.5
    a = torch.sigmoid(a0.float().reshape(1, 1, C) + a_lin.float())
    if v_first is not None:
        vf = vf + (v_first.float() - vf) * torch.sigmoid(v0.float().reshape(1, 1, C) + v_lin.float())
    kk = kf * k_k.float().reshape(1, 1, C)
    kk = F.normalize(kk.reshape(B, T, C // head_size, head_size), dim=-1, p=2.0).reshape(B, T, C)
    k_mod = kf * (1 + (a - 1) * k_a.float().reshape(1, 1, C))
    return w.to(dt), k_mod.to(dt), vf.to(dt), (-kk).to(dt), (kk * a).to(dt)


def gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size: int = 64, eps: float = GROUPNORM_EPS):
    """``(GroupNorm_H(y) + (sum_n r*k*r_k) * v) * g`` with one group per head."""
    dt = y.dtype
    B, T, C = y.shape
    H = C // head_size
    yn = F.group_norm(y.float().reshape(B * T, C), H, gn_w.float(), gn_b.float(), eps).reshape(B, T, C)
    rk = (r.float().reshape(B, T, H, -1) * k.float().reshape(B, T, H, -1) * r_k.float().reshape(H, -1)).sum(-1, keepdim=True)
    out = yn + (rk * v.float().reshape(B, T, H, -1)).reshape(B, T, C)
    return (out * g.float()).to(dt)


def relu_squared(x):
    return torch.relu(x) ** 2


# --------------------------------------------------------------------------- loss
class _L2Wrap(torch.autograd.Function):
    """Identity on the loss; adds ``factor * max_logit`` to the arg-max logit's gradient."""

    @staticmethod
    def forward(ctx, loss, logits, factor):
        ctx.save_for_backward(logits)
        ctx.factor = factor
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        (logits,) = ctx.saved_tensors
        maxx, ids = torch.max(logits, dim=-1, keepdim=True)
        gy = torch.zeros_like(logits)
        gy.scatter_(-1, ids, maxx * ctx.factor)
        return grad_output, gy, None


class L2Wrap:
    """``L2Wrap.apply(loss, logits)`` with ``logits [B, T, V]``: the stand-alone form of the regulariser that the
    fused head kernels apply in place (``rwkvtune/training/lightning_module.py:22-39``); factor ``1e-4 / (B * T)``."""

    @staticmethod
    def apply(loss: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        return _L2Wrap.apply(loss, logits, 1e-4 / (logits.shape[0] * logits.shape[1]))


def linear_cross_entropy(x, weight, labels, l2wrap: bool = True, ignore_index: int = -100,
                         l2wrap_tokens: Optional[int] = None):
    """``CrossEntropy(x @ weight^T, labels)`` averaged over non-ignored targets, plus L2Wrap.

    ``x`` is ``[M, C]``, ``weight`` ``[V, C]``, ``labels`` ``[M]``.  The L2Wrap
    factor is ``1e-4 / l2wrap_tokens`` with ``l2wrap_tokens`` defaulting to ``M``
    (the reference divides by ``B*T`` of the logits tensor).
    """
    logits = (x @ weight.t()).float()
    loss = F.cross_entropy(logits, labels, ignore_index=ignore_index)
    if l2wrap:
        n = l2wrap_tokens if l2wrap_tokens is not None else logits.shape[0]
        loss = _L2Wrap.apply(loss, logits, L2WRAP_FACTOR / n)
    return loss


def linear_logprob_entropy(x, weight, targets, temperature: float = 1.0, with_entropy: bool = True):
    """Per-row ``log_softmax(x @ weight^T / temperature)[target]`` and the entropy of that distribution."""
    logits = (x @ weight.t()).float()
    if temperature != 1.0:
        logits = logits / temperature
    lse = torch.logsumexp(logits, dim=-1)
    logp = logits.gather(-1, targets.unsqueeze(-1)).squeeze(-1) - lse
    ent = None
    if with_entropy:
        p = torch.softmax(logits, dim=-1)
        ent = lse - (p * logits).sum(-1)
    return logp, ent


# --------------------------------------------------------------------------- optimiser
def adamw_step(p32, g, m, v, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
               step: int, grad_scale: float = 1.0):
    """Decoupled-weight-decay Adam with bias correction on fp32 tensors, in place."""
    g = g.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    p32.mul_(1 - lr * weight_decay).addcdiv_(m, denom, value=-lr / bc1)
    return p32
