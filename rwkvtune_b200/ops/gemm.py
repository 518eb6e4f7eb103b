"""bf16 GEMM front-end.

Three layouts cover everything the network needs (``x`` is always ``[M, K]`` row-major):

* ``mm_nt(x, w)``  = ``x @ w^T``  with ``w [N, K]``  (``nn.Linear`` forward, dgrad of the low-rank maps)
* ``mm_nn(x, w)``  = ``x @ w``    with ``w [K, N]``  (low-rank maps forward, ``nn.Linear`` dgrad)
* ``mm_tn(a, b)``  = ``a^T @ b``  with ``a [M, N1]``, ``b [M, N2]``  (every weight gradient)

``linear`` / ``matmul`` wrap them in autograd.  The tcgen05 kernels of
``rwkvtune_b200/csrc/gemm_tcgen05.cu`` serve the shapes they support (see ``native_ok``);
other shapes go to the library GEMM.
"""
from __future__ import annotations

import torch

_USE_NATIVE = True


def set_native(enabled: bool) -> None:
    global _USE_NATIVE
    _USE_NATIVE = bool(enabled)


def _native():
    if not _USE_NATIVE:
        return None
    try:
        from . import gemm_native
    except ImportError:
        return None
    return gemm_native


def mm_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    n = _native()
    if n is not None:
        if n.SMALL_M_DISPATCH and n.small_m_ok(x, w):
            return n.small_m_group([x], [w])[0]
        if n.native_ok(x, w, "nt"):
            return n.mm_nt(x, w)
    return x @ w.t()


def linear_group(xs, ws):
    """``[x_i @ w_i^T]`` for several independent projections with the same row count.  During decoding
    (few rows, no autograd) they go out as one grouped launch; otherwise one ``linear`` each."""
    n = _native()
    if (n is not None and n.SMALL_M_DISPATCH and not torch.is_grad_enabled() and len(xs) <= 8
            and all(x.shape[:-1] == xs[0].shape[:-1] for x in xs)):
        x2 = [x.reshape(-1, x.shape[-1]) for x in xs]
        if all(n.small_m_ok(a, w) for a, w in zip(x2, ws)):
            ys = n.small_m_group(x2, list(ws))
            return [y.reshape(*x.shape[:-1], w.shape[0]) for y, x, w in zip(ys, xs, ws)]
    return [linear(x, w) for x, w in zip(xs, ws)]


def mm_nn(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    n = _native()
    if n is not None and n.native_ok(x, w, "nn"):
        return n.mm_nn(x, w)
    return x @ w


def _acc_ok(n, y: torch.Tensor) -> bool:
    return (n is not None and y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.stride(1) == 1
            and y.data_ptr() % 16 == 0 and (y.stride(0) * 2) % 16 == 0)


def addmm_nt_(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y += x @ w^T`` in place; on the native path the sum happens in the GEMM epilogue (no temporary)."""
    n = _native()
    if _acc_ok(n, y) and n.native_ok(x, w, "nt"):
        return n.mm_nt(x, w, out=y)
    return y.add_(x @ w.t())


def addmm_nn_(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y += x @ w`` in place (see :func:`addmm_nt_`)."""
    n = _native()
    if _acc_ok(n, y) and n.native_ok(x, w, "nn"):
        return n.mm_nn(x, w, out=y)
    return y.add_(x @ w)


def addmm_tn_(y: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``y += a^T @ b`` in place (a weight gradient accumulated over row slabs; see :func:`addmm_nt_`)."""
    n = _native()
    if _acc_ok(n, y) and n.native_ok(a, b, "tn"):
        return n.mm_tn(a, b, out=y)
    return y.add_((a.t() @ b).to(y.dtype))


def mm_tn_into(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``out = a^T @ b`` written into an existing bf16 ``[M, N]`` buffer (a weight gradient formed directly in a
    communication staging buffer)."""
    n = _native()
    if _acc_ok(n, out) and n.native_ok(a, b, "tn"):
        return n.mm_tn(a, b, out=out, accumulate=False)
    return out.copy_((a.t() @ b).to(out.dtype))


def mm_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    n = _native()
    if n is not None:
        if n.native_ok(a, b, "tn"):
            return n.mm_tn(a, b)
        splits = n.splitk_plan(a, b)
        if splits:
            return n.mm_tn_splitk(a, b, splits)
    return a.t() @ b


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        return mm_nt(x2, w).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = mm_nn(dy2, w).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            dw = mm_tn(dy2, x.reshape(-1, x.shape[-1]))
        return dx, dw


class _LinearAdd(torch.autograd.Function):
    """``residual + x @ w^T`` with the sum formed in the GEMM epilogue (residual stream update of a block)."""

    @staticmethod
    def forward(ctx, x, w, residual):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, residual.shape[-1])
        n = _native()
        if _acc_ok(n, r2) and n.native_ok(x2, w, "nt"):
            y = n.mm_nt(x2, w, residual=r2)
        else:
            y = r2 + mm_nt(x2, w)
        return y.reshape(residual.shape)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = mm_nn(dy2, w).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            dw = mm_tn(dy2, x.reshape(-1, x.shape[-1]))
        return dx, dw, (dy if ctx.needs_input_grad[2] else None)


def linear_add(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    return _LinearAdd.apply(x, w, residual)


class _MatMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        return mm_nn(x2, w).reshape(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = mm_nt(dy2, w).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            dw = mm_tn(x.reshape(-1, x.shape[-1]), dy2)
        return dx, dw


class _MatMulAct(torch.autograd.Function):
    """``act(x @ w)`` for ``act`` in tanh / sigmoid, the activation applied in the GEMM epilogue; the backward
    needs only the output (``tanh' = 1 - y^2``, ``sigmoid' = y (1 - y)``)."""

    @staticmethod
    def forward(ctx, x, w, act: str):
        x2 = x.reshape(-1, x.shape[-1])
        n = _native()
        if n is not None and n.native_ok(x2, w, "nn"):
            y = n.mm_nn(x2, w, epilogue=3 if act == "tanh" else 4)
        else:
            y = torch.tanh(x2 @ w) if act == "tanh" else torch.sigmoid(x2 @ w)
        ctx.save_for_backward(x, w, y)
        ctx.act = act
        return y.reshape(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x, w, y = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dpre = dy2 * (1 - y * y) if ctx.act == "tanh" else dy2 * (y * (1 - y))
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = mm_nt(dpre, w).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            dw = mm_tn(x.reshape(-1, x.shape[-1]), dpre)
        return dx, dw, None


def matmul_act(x, w, act: str):
    if act not in ("tanh", "sigmoid"):
        raise ValueError(f"unsupported activation {act!r}")
    return _MatMulAct.apply(x, w, act)


def linear(x, weight):
    return _Linear.apply(x, weight)


def matmul(x, w):
    return _MatMul.apply(x, w)
