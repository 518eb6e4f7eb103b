"""Operator entry points with the call conventions of ``rwkvtune/models/rwkv7/operators`` (``wkv_loader.py:162-620``,
``wkv_infctx.py:156-200``, ``wkv_cpu.py:9-80``).

Nothing is compiled or loaded here: every function forwards to :func:`rwkvtune_b200.ops.wkv7`, which runs the
ahead-of-time built sm_100a kernels on CUDA tensors and the plain PyTorch recurrence on CPU tensors.  The loaders
exist so that code written against the reference's ``load_wkv_operator`` / ``rwkv7_wkv`` keeps working.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from .... import ops
from ....ops import reference as _reference
from .infctx_oracle import (RWKV7InfctxNaiveFunction, WKV7InfctxFunction, naive_recurrent_rwkv7_bwd,
                            naive_recurrent_rwkv7_fwd)

__all__ = ["load_wkv_operator", "rwkv7_wkv", "load_wkv7_operator", "load_cpu_operator", "load_cuda_operator_train",
           "load_cuda_operator_inference", "load_cuda_operator_infctx", "rwkv7_wkv_cpu", "rwkv7_wkv_infctx",
           "rwkv7_wkv_infctx_naive", "naive_recurrent_rwkv7_fwd", "naive_recurrent_rwkv7_bwd",
           "RWKV7InfctxNaiveFunction", "WKV7InfctxFunction"]


def _stateful(head_size: int) -> Callable:
    def op(r, w, k, v, a, b, state: Optional[torch.Tensor] = None, return_state: bool = False):
        y, s = ops.wkv7(r, w, k, v, a, b, head_size, state, return_state)
        return (y, s) if return_state else y

    return op


def load_cpu_operator(head_size: int = 64) -> Callable:
    """``op(r, w, k, v, a, b, state=None, return_state=False)`` on CPU tensors ``[B, T, C]``."""
    def op(r, w, k, v, a, b, state: Optional[torch.Tensor] = None, return_state: bool = False):
        y, s = _reference.wkv7(r, w, k, v, a, b, head_size, state)
        y = y.to(r.dtype)
        return (y, s) if return_state else y

    return op


def load_cuda_operator_train(head_size: int = 64) -> Callable:
    """``op(r, w, k, v, a, b) -> y``, differentiable in all six inputs."""
    def op(r, w, k, v, a, b):
        return ops.wkv7(r, w, k, v, a, b, head_size)[0]

    return op


def load_cuda_operator_inference(head_size: int = 64) -> Callable:
    """``op(r, w, k, v, a, b, state, return_state)`` with an fp32 state ``[B, H, N, N]``."""
    return _stateful(head_size)


def load_wkv_operator(device: str = "cuda", for_inference: bool = False, head_size: int = 64) -> Callable:
    if device == "cpu":
        return load_cpu_operator(head_size)
    if device == "cuda":
        return load_cuda_operator_inference(head_size) if for_inference else load_cuda_operator_train(head_size)
    raise ValueError(f"unsupported device {device!r}: expected 'cpu' or 'cuda'")


load_wkv7_operator = load_wkv_operator


def rwkv7_wkv(q, w, k, v, a, b, head_size: int = 64, state: Optional[torch.Tensor] = None, return_state: bool = False):
    """``[B, T, C]`` inputs; returns ``y`` or ``(y, final_state)`` when ``return_state``."""
    return _stateful(head_size)(q, w, k, v, a, b, state, return_state)


def rwkv7_wkv_cpu(r, w, k, v, a, b, HEAD_SIZE: int = 64, state: Optional[torch.Tensor] = None):
    """The fp32 oracle; accepts ``[T, C]`` or ``[B, T, C]`` and always returns ``(y, final_state)``."""
    squeeze = r.dim() == 2
    if squeeze:
        r, w, k, v, a, b = (t.unsqueeze(0) for t in (r, w, k, v, a, b))
        state = None if state is None else state.unsqueeze(0)
    y, s = _reference.wkv7(r, w, k, v, a, b, HEAD_SIZE, state)
    return (y.squeeze(0), s.squeeze(0)) if squeeze else (y, s)


def _infctx(fn, w, q, k, v, a, b, state, scale):
    B, T, H, N = q.shape
    flat = lambda t: t.reshape(B, T, H * N)   # noqa: E731
    qq = q * scale if scale != 1.0 else q
    y, s = fn(flat(qq), flat(w), flat(k), flat(v), flat(a), flat(b), N, state)
    return y.reshape(B, T, H, N).to(q.dtype), s


def rwkv7_wkv_infctx(w, q, k, v, a, b, state: Optional[torch.Tensor] = None,
                     scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk step of infinite-context training: ``[B, T, H, N]`` inputs (note the argument order, ``w`` first;
    decay ``exp(-exp(w))`` as everywhere else), state ``[B, H, N, N]`` in and out, gradients through the inputs and
    the state."""
    return _infctx(lambda *args: ops.wkv7(*args, True), w, q, k, v, a, b, state, scale)


def rwkv7_wkv_infctx_naive(q, k, v, w, a, b, state: Optional[torch.Tensor] = None,
                           scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """The oracle of the chunk step: fp32 step-by-step recurrence with a closed-form backward (no autograd tape).
    Note the argument order, ``q, k, v, w`` — that of ``wkv_infctx_naive.py:228-250``, not of
    :func:`rwkv7_wkv_infctx`.  Returns fp32 ``(output [B, T, H, N], final_state [B, H, N, N])``."""
    return RWKV7InfctxNaiveFunction.apply(q, k, v, w, a, b, scale, state)


def load_cuda_operator_infctx():
    """The reference returns a compiled module here; this returns the chunk-step function itself."""
    return rwkv7_wkv_infctx
