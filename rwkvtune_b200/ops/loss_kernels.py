"""Head GEMM fused with selective log-softmax and entropy (GRPO log-probabilities).

Replaces ``selective_log_softmax`` and ``entropy_from_logits``
(``rwkvtune/training/grpo/utils.py:13-152``) applied to materialised ``[n, L, V]`` logits: rows
are processed in slabs and the backward pass recomputes each slab instead of saving it.
"""
from __future__ import annotations

import torch

from . import gemm

SLAB = 4096


def _rows_native(x, weight) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0


class _LogprobEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, targets, temperature, with_entropy):
        M = x.shape[0]
        logp = torch.empty(M, dtype=torch.float32, device=x.device)
        ent = torch.empty(M, dtype=torch.float32, device=x.device) if with_entropy else None
        inv_t = 1.0 / temperature
        native = _rows_native(x, weight)
        if native:
            from ._ext import call, f32, i32, i64, ptr, stream
            targets = targets.contiguous().long()
        for s in range(0, M, SLAB):
            e = min(M, s + SLAB)
            if native:   # statistics in one sweep over the bf16 slab
                z = gemm.mm_nt(x[s:e], weight).contiguous()
                call("rwkv_logprob_entropy_rows_fwd", ptr(z), ptr(targets[s:e]), f32(inv_t), ptr(logp[s:e]),
                     ptr(ent[s:e] if with_entropy else None), i64(e - s), i32(z.shape[1]), stream())
                continue
            z = gemm.mm_nt(x[s:e], weight).float() * inv_t
            lse = torch.logsumexp(z, dim=-1)
            logp[s:e] = z.gather(-1, targets[s:e, None]).squeeze(-1) - lse
            if with_entropy:
                p = torch.exp(z - lse[:, None])
                ent[s:e] = lse - (p * z).sum(-1)
        ctx.save_for_backward(x, weight, targets)
        ctx.inv_t = inv_t
        ctx.with_entropy = with_entropy
        if with_entropy:
            return logp, ent
        ctx.mark_non_differentiable()
        return logp, None

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        x, weight, targets = ctx.saved_tensors
        M = x.shape[0]
        inv_t = ctx.inv_t
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=x.device) if ctx.needs_input_grad[1] else None
        native = _rows_native(x, weight)
        if native:
            from ._ext import call, f32, i32, i64, ptr, stream
            targets = targets.contiguous().long()
            gl_all = None if g_logp is None else g_logp.float().contiguous()
            ge_all = None if (g_ent is None or not ctx.with_entropy) else g_ent.float().contiguous()
        for s in range(0, M, SLAB):
            e = min(M, s + SLAB)
            if native:   # recompute the slab, rewrite it in place as d logits
                dz = gemm.mm_nt(x[s:e], weight).contiguous()
                call("rwkv_logprob_entropy_rows_bwd", ptr(dz), ptr(targets[s:e]), f32(inv_t),
                     ptr(None if gl_all is None else gl_all[s:e]), ptr(None if ge_all is None else ge_all[s:e]),
                     i64(e - s), i32(dz.shape[1]), stream())
            else:
                z = gemm.mm_nt(x[s:e], weight).float() * inv_t
                lse = torch.logsumexp(z, dim=-1, keepdim=True)
                p = torch.exp(z - lse)
                gl = g_logp[s:e, None].float() if g_logp is not None else torch.zeros_like(lse)
                dz = -p * gl
                dz.scatter_add_(-1, targets[s:e, None], gl)
                if ctx.with_entropy and g_ent is not None:
                    h = lse - (p * z).sum(-1, keepdim=True)
                    dz -= g_ent[s:e, None].float() * p * (z - lse + h)
                dz = (dz * inv_t).to(x.dtype)
            if dx is not None:
                dx[s:e] = gemm.mm_nn(dz, weight)
            if dw is not None:
                dw += gemm.mm_tn(dz, x[s:e]).float()
        return dx, (None if dw is None else dw.to(weight.dtype)), None, None, None


def linear_logprob_entropy(x, weight, targets, temperature: float = 1.0, with_entropy: bool = True):
    return _LogprobEntropy.apply(x, weight, targets, temperature, with_entropy)
