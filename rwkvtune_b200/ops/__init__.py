"""Fused operator entry points.

Every function here has two implementations with one contract:

* CUDA tensors run the hand-written sm_100a kernels from ``rwkvtune_b200/csrc``
  (loaded through :mod:`rwkvtune_b200.ops._ext`).  If the native library is
  missing, a CUDA call raises instead of silently running something else.
* CPU tensors run the plain-PyTorch statements in :mod:`rwkvtune_b200.ops.reference`,
  which are also the oracles of the kernel tests.

``set_kernel_enabled(name, False)`` routes one operator family to the PyTorch
statement on the GPU as well; it exists for A/B measurements and for bisecting
numerical differences, not as a production mode.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from . import reference
from .reference import GROUPNORM_EPS, LAYERNORM_EPS, L2WRAP_FACTOR

_KERNELS: Dict[str, bool] = {
    "wkv7": True,
    "ln_shift_mix": True,
    "layer_norm": True,
    "timemix_prep": True,
    "gn_bonus_gate": True,
    "relu_squared": True,
    "linear_cross_entropy": True,
    "linear_logprob_entropy": True,
    "gemm": True,
    "gather": True,
}


def param_epoch() -> int:
    """Counter bumped whenever parameters are rewritten by the optimiser kernels."""
    from . import cuda_ops_epoch

    return cuda_ops_epoch.EPOCH[0]


def bump_param_epoch() -> None:
    from . import cuda_ops_epoch

    cuda_ops_epoch.EPOCH[0] += 1
    try:
        from . import cuda_ops

        cuda_ops.bump_param_epoch()
    except Exception:
        pass


def set_kernel_enabled(name: str, enabled: bool) -> None:
    if name not in _KERNELS:
        raise KeyError(f"unknown kernel family {name!r}; known: {sorted(_KERNELS)}")
    _KERNELS[name] = bool(enabled)


def kernel_enabled(name: str) -> bool:
    return _KERNELS[name]


def _native(t: torch.Tensor, name: str) -> bool:
    return t.is_cuda and _KERNELS[name]


def _cuda():
    from . import cuda_ops  # imported lazily: needs the native library

    return cuda_ops


# ------------------------------------------------------------------------------- GEMMs
def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight^T`` for an ``nn.Linear`` weight ``[out, in]``."""
    if _native(x, "gemm"):
        return _cuda().linear(x, weight)
    return torch.nn.functional.linear(x, weight)


def matmul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w`` for a right-multiplied ``[in, out]`` matrix (the low-rank adapters)."""
    if _native(x, "gemm"):
        return _cuda().matmul(x, w)
    return x @ w


def matmul_act(x: torch.Tensor, w: torch.Tensor, act: str) -> torch.Tensor:
    """``tanh(x @ w)`` or ``sigmoid(x @ w)`` (first stage of the low-rank decay / gate chains); the activation runs
    in the GEMM epilogue on CUDA."""
    if _native(x, "gemm") and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from . import gemm

        return gemm.matmul_act(x, w, act)
    pre = x @ w
    return torch.tanh(pre) if act == "tanh" else torch.sigmoid(pre)


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """``residual + x @ weight^T``; on CUDA the residual is added in the GEMM epilogue."""
    if _native(x, "gemm") and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        from . import gemm

        return gemm.linear_add(x, weight, residual)
    return residual + torch.nn.functional.linear(x, weight)


def channel_mix_ffn(xk: torch.Tensor, w_key: torch.Tensor, w_value: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """``residual + relu(xk @ w_key^T)^2 @ w_value^T`` (the feed-forward half of a block) as one autograd node."""
    if _native(xk, "gemm") and _native(xk, "relu_squared"):
        return _cuda().channel_mix_ffn(xk, w_key, w_value, residual)
    hidden = reference.relu_squared(torch.nn.functional.linear(xk, w_key))
    return residual + torch.nn.functional.linear(hidden, w_value)


def linear_group(xs, weights):
    """Several independent ``x_i @ W_i^T`` with the same leading shape; one grouped launch while decoding."""
    if _native(xs[0], "gemm"):
        from . import gemm

        return gemm.linear_group(list(xs), list(weights))
    return [torch.nn.functional.linear(x, w) for x, w in zip(xs, weights)]


def projections_with_lowrank(lin_xs, lin_ws, lr_xs, lr_w1, lr_acts, lr_w2):
    """``([x @ W^T ...], [act(x @ w1) @ w2 ...])``: the ``nn.Linear`` projections and the low-rank chains of a
    time-mix block (``rwkvtune/models/rwkv7/model.py:146-160``).  ``lr_acts[i]`` is ``None``, ``"tanh"`` or
    ``"sigmoid"``.  While decoding on CUDA the whole set is two grouped launches."""
    if _native((list(lin_xs) + list(lr_xs))[0], "gemm"):
        from . import gemm

        return gemm.projections_with_lowrank(lin_xs, lin_ws, lr_xs, lr_w1, lr_acts, lr_w2)
    act = {None: lambda t: t, "tanh": torch.tanh, "sigmoid": torch.sigmoid}
    return ([torch.nn.functional.linear(x, w) for x, w in zip(lin_xs, lin_ws)],
            [act[a](x @ w1) @ w2 for x, w1, a, w2 in zip(lr_xs, lr_w1, lr_acts, lr_w2)])


def decode_projection_set(lin, lowrank=(), prefetch=None):
    """Independent projections of the same few rows (a decode step) in at most two grouped launches, or ``None`` when
    the set does not qualify (CPU tensors, autograd recording, more than 128 rows, odd shapes): see
    ``ops/gemm.py::decode_projection_set`` for the argument format."""
    if lin and _native(lin[0][0], "gemm") or (not lin and lowrank and _native(lowrank[0][0], "gemm")):
        from . import gemm

        return gemm.decode_projection_set(list(lin), list(lowrank), prefetch)
    return None


def linear_relu_sq(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``relu(x @ weight^T) ** 2`` (channel-mix key projection); fused into the GEMM epilogue on CUDA."""
    if _native(x, "gemm") and _native(x, "relu_squared"):
        return _cuda().linear_relu_sq(x, weight)
    return reference.relu_squared(torch.nn.functional.linear(x, weight))


# ------------------------------------------------------------------------------- fused element-wise
def layer_norm(x, weight, bias, eps: float = LAYERNORM_EPS):
    if _native(x, "layer_norm"):
        return _cuda().layer_norm(x, weight, bias, eps)
    return reference.layer_norm(x, weight, bias, eps)


def ln_shift_mix(x, ln_w, ln_b, mix, prev=None, eps: float = LAYERNORM_EPS):
    if _native(x, "ln_shift_mix"):
        return _cuda().ln_shift_mix(x, ln_w, ln_b, mix, prev, eps)
    return reference.ln_shift_mix(x, ln_w, ln_b, mix, prev, eps)


def ln_shift_mix_unbound(x, ln_w, ln_b, mix, prev=None, eps: float = LAYERNORM_EPS):
    """:func:`ln_shift_mix` with the mixed outputs as a tuple of ``K`` tensors (no stacked gradient in backward).

    Returns ``(outs, last_row, x)``.  The third item is ``x`` again; a residual connection that adds to *it*
    sends its gradient through this operator's backward kernel, which sums it into ``dx`` for free."""
    if _native(x, "ln_shift_mix"):
        return _cuda().ln_shift_mix_unbound(x, ln_w, ln_b, mix, prev, eps)
    outs, last = reference.ln_shift_mix(x, ln_w, ln_b, mix.reshape(-1, x.shape[-1]), prev, eps)
    return outs.unbind(0), last, x


def timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, head_size: int = 64):
    if _native(k, "timemix_prep"):
        return _cuda().timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, head_size)
    return reference.timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, w0, a0, v0, k_k, k_a, head_size)


def gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size: int = 64, eps: float = GROUPNORM_EPS):
    if _native(y, "gn_bonus_gate"):
        return _cuda().gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size, eps)
    return reference.gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size, eps)


def relu_squared(x):
    if _native(x, "relu_squared"):
        return _cuda().relu_squared(x)
    return reference.relu_squared(x)


# ------------------------------------------------------------------------------- recurrence
def wkv7(r, w, k, v, a, b, head_size: int = 64, state: Optional[torch.Tensor] = None,
         return_state: bool = False):
    """WKV7 recurrence.  Returns ``(y, final_state or None)``; ``y`` has the dtype of ``r``."""
    if _native(r, "wkv7"):
        return _cuda().wkv7(r, w, k, v, a, b, head_size, state, return_state)
    if r.device.type == "cpu":      # one autograd node with a closed-form backward instead of the traced statement
        from . import cpu_ops

        y, s = cpu_ops.wkv7(r, w, k, v, a, b, head_size, state)
    else:
        y, s = reference.wkv7(r, w, k, v, a, b, head_size, state)
    return y.to(r.dtype), (s if return_state else None)


def wkv7_pool_step(r, w, k, v, a, b, pool: torch.Tensor, slots: torch.Tensor, head_size: int = 64) -> torch.Tensor:
    """WKV7 forward without autograd on a state pool ``[n_slots, H, N, N]`` (fp32): sequence ``i`` reads and writes
    ``pool[slots[i]]`` in place.  ``slots`` must be distinct."""
    if _native(r, "wkv7") and head_size == 64:
        return _cuda().wkv7_pool_step(r, w, k, v, a, b, pool, slots)
    with torch.no_grad():
        if r.device.type == "cpu":
            from . import cpu_ops

            y, s = cpu_ops.wkv7(r, w, k, v, a, b, head_size, pool.index_select(0, slots))
        else:
            y, s = reference.wkv7(r, w, k, v, a, b, head_size, pool.index_select(0, slots))
        pool.index_copy_(0, slots, s.to(pool.dtype))
    return y.to(r.dtype)


def timemix_decode_core_ok(r, g, state, head_size: int = 64) -> bool:
    """True when :func:`timemix_decode_core` applies: CUDA, one token per sequence, bf16, head size 64, an existing fp32
    state, no autograd, and none of the three kernels it replaces switched off."""
    if not (_native(r, "wkv7") and _native(r, "timemix_prep") and _native(r, "gn_bonus_gate")):
        return False
    return _cuda().timemix_decode_core_ok(r, g, state, head_size)


def timemix_decode_core(r, k, v, v_first, w_lin, a_lin, v_lin, g, w0, a0, v0, k_k, k_a, r_k, gn_w, gn_b, state,
                        eps: float = GROUPNORM_EPS):
    """One decoding step of a block's recurrent core - ``timemix_prep``, the WKV7 update and ``gn_bonus_gate`` - as a
    single kernel (check :func:`timemix_decode_core_ok` first).  Returns ``(z, new_state)``."""
    return _cuda().timemix_decode_core(r, k, v, v_first, w_lin, a_lin, v_lin, g, w0, a0, v0, k_k, k_a, r_k, gn_w, gn_b,
                                       state, eps)


def wkv7_gn(r, w, k, v, a, b, g, gn_w, gn_b, r_k, head_size: int = 64, state: Optional[torch.Tensor] = None,
            return_state: bool = False, eps: float = GROUPNORM_EPS):
    """The recurrence followed by GroupNorm + bonus + gate; returns ``(z, final_state or None)``.  On CUDA the two
    share one autograd node so that the gradients of ``r``, ``k``, ``v`` are summed inside the backward kernel."""
    if _native(r, "wkv7") and _native(r, "gn_bonus_gate") and not isinstance(state, tuple):
        return _cuda().wkv7_gn(r, w, k, v, a, b, g, gn_w, gn_b, r_k, head_size, state, return_state, eps)
    if isinstance(state, tuple):
        y, s = wkv7_pool_step(r, w, k, v, a, b, state[0], state[1], head_size), state
    else:
        y, s = wkv7(r, w, k, v, a, b, head_size, state, return_state)
    return gn_bonus_gate(y, r, k, v, g, gn_w, gn_b, r_k, head_size, eps), s


# ------------------------------------------------------------------------------- losses
def linear_cross_entropy(x, weight, labels, l2wrap: bool = True, ignore_index: int = -100,
                         l2wrap_tokens: Optional[int] = None):
    if _native(x, "linear_cross_entropy"):
        return _cuda().linear_cross_entropy(x, weight, labels, l2wrap, ignore_index, l2wrap_tokens)
    return reference.linear_cross_entropy(x, weight, labels, l2wrap, ignore_index, l2wrap_tokens)


def linear_logprob_entropy(x, weight, targets, temperature: float = 1.0, with_entropy: bool = True):
    if _native(x, "linear_logprob_entropy"):
        return _cuda().linear_logprob_entropy(x, weight, targets, temperature, with_entropy)
    return reference.linear_logprob_entropy(x, weight, targets, temperature, with_entropy)


# ------------------------------------------------------------------------------- gathers
def embedding(idx: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Embedding lookup; the gradient accumulates repeated tokens in fp32 in a fixed order."""
    if _native(weight, "gather"):
        return _cuda().embedding(idx, weight)
    return torch.nn.functional.embedding(idx, weight)


def gather_rows(src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """``src.index_select(0, index)``: state fan-out to sampling paths and compaction of live rows."""
    if _native(src, "gather"):
        return _cuda().gather_rows(src, index)
    return src.index_select(0, index)
