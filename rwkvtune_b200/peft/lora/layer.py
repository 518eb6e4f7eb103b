"""LoRA-wrapped linear layer with a fused forward/backward.

``y = x W^T + s (x A^T) B^T`` with the base weight frozen.  The reference evaluates this as three
``F.linear`` calls and lets autograd also differentiate through the base layer
(``rwkvtune/peft/lora/layer.py:92-130``).  Here one autograd node does it: the backward produces
``dx = dy W + s (dy B) A``, ``dA`` and ``dB`` and never forms the (unused) base weight gradient.  Both ``y`` and ``dx``
are single GEMM launches: the rank-``r`` term is appended to the contraction of the base product (``[x | s x A^T]`` against
``[W | B]``), the second operand pair being fetched through its own TMA tensor maps.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ...ops import gemm


def _relu_sq_grad(y: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """Gradient of ``relu(p)^2`` with respect to ``p`` expressed through its output ``y``: ``dy * 2 sqrt(y)``."""
    if y.is_cuda and y.dtype == torch.bfloat16 and y.numel() % 8 == 0:
        from ...ops import _ext

        if _ext.available():
            dyc = dy if dy.is_contiguous() else dy.contiguous()
            out = torch.empty_like(y)
            _ext.call("rwkv_relu_sq_backward", _ext.ptr(y), _ext.ptr(dyc), _ext.ptr(out), _ext.i64(y.numel()), _ext.i32(1),
                      _ext.stream())
            return out
    return (dy.float() * 2.0 * y.float().sqrt()).to(dy.dtype)


class _LoraLinearFn(torch.autograd.Function):
    """``act(x W^T + s (x A^T) B^T) + residual`` (``act`` = identity or relu^2; a residual only without activation)."""

    @staticmethod
    def forward(ctx, x, w, a, b, scaling: float, w_needs_grad: bool, residual=None, act=None):
        x2 = x.reshape(-1, x.shape[-1])
        xa_s = gemm.mm_nt(x2, a) * scaling           # [M, r], scaled once: used by the forward and by dB
        r2 = None if residual is None else residual.reshape(-1, residual.shape[-1])
        # the product with B rides as the last K block of the base GEMM (one launch, no read-modify-write of y);
        # activation or residual sum in the same launch's epilogue
        y = gemm.mm_nt_plus(x2, w, xa_s, b, act=act, residual=r2)
        ctx.save_for_backward(x2, w, a, b, xa_s, y if act else None)
        ctx.scaling, ctx.shape, ctx.act = scaling, x.shape, act
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, a, b, xa_s, y = ctx.saved_tensors
        s = ctx.scaling
        dy2 = dy.reshape(-1, dy.shape[-1])
        dpre = _relu_sq_grad(y, dy2) if ctx.act else dy2
        dyb_s = gemm.mm_nn(dpre, b) * s              # [M, r], scaled once: used by dx and by dA
        dx = dw = da = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm.mm_nn_plus(dpre, w, dyb_s, a).reshape(ctx.shape)
        if ctx.needs_input_grad[1]:
            dw = gemm.mm_tn(dpre, x2)
        if ctx.needs_input_grad[2]:
            da = gemm.mm_tn(dyb_s, x2)
        if ctx.needs_input_grad[3]:
            db = gemm.mm_tn(dpre, xa_s)
        d_res = dy if (len(ctx.needs_input_grad) > 6 and ctx.needs_input_grad[6]) else None
        return dx, dw, da, db, None, None, d_res, None


class LoraLinear(nn.Module):
    def __init__(self, base_layer: nn.Linear, r: int = 64, lora_alpha: int = 128, lora_dropout: float = 0.0,
                 use_rslora: bool = False, init_lora_weights=True):
        super().__init__()
        if not isinstance(base_layer, nn.Linear):
            raise TypeError("LoraLinear wraps nn.Linear modules only")
        self.base_layer = base_layer
        self.in_features, self.out_features = base_layer.in_features, base_layer.out_features
        self.r, self.lora_alpha = r, lora_alpha
        self.scaling = lora_alpha / math.sqrt(r) if use_rslora else lora_alpha / r
        dev, dt = base_layer.weight.device, base_layer.weight.dtype
        self.lora_A = nn.Parameter(torch.zeros(r, self.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, r, device=dev, dtype=dt))
        self.lora_dropout = nn.Dropout(lora_dropout) if lora_dropout > 0 else nn.Identity()
        if init_lora_weights:
            self.reset_lora_parameters(init_lora_weights)
        self.merged = False
        self.disabled = False

    @property
    def weight(self) -> torch.Tensor:
        return self.base_layer.weight

    def reset_lora_parameters(self, mode=True) -> None:
        if mode == "gaussian":
            nn.init.normal_(self.lora_A, std=1.0 / self.r)
        else:
            a = torch.empty(self.lora_A.shape, dtype=torch.float32, device=self.lora_A.device)
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
            with torch.no_grad():
                self.lora_A.copy_(a)
        nn.init.zeros_(self.lora_B)

    def effective_weight(self) -> torch.Tensor:
        if self.merged or self.disabled:
            return self.base_layer.weight
        return self.base_layer.weight + (self.lora_B @ self.lora_A) * self.scaling

    def forward(self, x: torch.Tensor, residual: torch.Tensor = None, act: str = None) -> torch.Tensor:
        """``act(base(x) + adapter(x)) + residual``; ``act`` is ``None`` or ``"relu_sq"`` (never with a residual).  On
        the training path both ride in the epilogue of the single fused GEMM launch."""
        if act is not None and residual is not None:
            raise ValueError("LoraLinear: an activation and a residual cannot be combined")
        sw = getattr(self, "_sharded", None)
        if sw is not None and not self.disabled and not (isinstance(self.lora_dropout, nn.Dropout) and self.training):
            from ...parallel.zero3 import lora_ag_linear     # ZeRO-3: the same fusion inside the all-gather GEMM

            return lora_ag_linear(x, sw, self.lora_A, self.lora_B, self.scaling, residual, act)
        fused = (sw is None and not (self.disabled or self.merged)
                 and not (not torch.is_grad_enabled() and x.is_cuda and x.numel() // x.shape[-1] <= 256)
                 and not (isinstance(self.lora_dropout, nn.Dropout) and self.training))
        if fused:
            return _LoraLinearFn.apply(x, self.base_layer.weight, self.lora_A, self.lora_B, self.scaling,
                                       self.base_layer.weight.requires_grad, residual, act)
        y = self._plain_forward(x)
        if act == "relu_sq":
            from ... import ops

            y = ops.relu_squared(y)
        return y if residual is None else residual + y

    def _plain_forward(self, x: torch.Tensor) -> torch.Tensor:
        sw = getattr(self, "_sharded", None)
        if sw is not None:   # ZeRO-3 sharded frozen base weight
            from ...parallel.zero3 import ag_linear, lora_ag_linear

            if self.disabled:
                return ag_linear(x, sw)
            return lora_ag_linear(x, sw, self.lora_A, self.lora_B, self.scaling)
        if self.disabled or self.merged:
            return self.base_layer(x)
        if not torch.is_grad_enabled() and x.is_cuda and x.numel() // x.shape[-1] <= 256:
            # decode-sized batch outside the grouped path: three library GEMMs, the adapter product added by the last one
            x2 = x.reshape(-1, x.shape[-1])
            y = torch.addmm(x2 @ self.base_layer.weight.t(), x2 @ self.lora_A.t(), self.lora_B.t(), alpha=self.scaling)
            return y.reshape(*x.shape[:-1], self.out_features)
        base = self.base_layer(x)
        xd = self.lora_dropout(x)
        return base + gemm.linear(gemm.linear(xd, self.lora_A), self.lora_B) * self.scaling

    def decode_spec(self):
        """``(weight, adapter)`` for the grouped decode path: ``adapter`` is ``None`` (merged or disabled) or
        ``(lora_A, lora_B, scaling)``.  ``None`` when the layer cannot take that path (sharded base, active dropout)."""
        if getattr(self, "_sharded", None) is not None:
            return None
        if self.merged or self.disabled:
            return self.base_layer.weight, None
        if isinstance(self.lora_dropout, nn.Dropout) and self.training:
            return None
        return self.base_layer.weight, (self.lora_A, self.lora_B, self.scaling)

    @torch.no_grad()
    def merge(self) -> None:
        if not self.merged:
            self.base_layer.weight.add_(((self.lora_B.float() @ self.lora_A.float()) * self.scaling).to(self.base_layer.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self) -> None:
        if self.merged:
            self.base_layer.weight.sub_(((self.lora_B.float() @ self.lora_A.float()) * self.scaling).to(self.base_layer.weight.dtype))
            self.merged = False

    def disable_adapter(self) -> None:
        self.disabled = True

    def enable_adapter(self) -> None:
        self.disabled = False

    def get_lora_state_dict(self) -> dict:
        return {"lora_A": self.lora_A.detach().clone(), "lora_B": self.lora_B.detach().clone()}

    def load_lora_state_dict(self, state_dict: dict) -> None:
        with torch.no_grad():
            if "lora_A" in state_dict:
                self.lora_A.copy_(state_dict["lora_A"])
            if "lora_B" in state_dict:
                self.lora_B.copy_(state_dict["lora_B"])

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, r={self.r}, "
                f"scaling={self.scaling:.4f}, merged={self.merged}, disabled={self.disabled}")
