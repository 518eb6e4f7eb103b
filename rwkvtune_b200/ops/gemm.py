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


def _decode(n) -> bool:
    return n is not None and n.DECODE_DISPATCH


def decode_products(xs, ws, acts=None, kn=None, residuals=None, prefetch=None):
    """``[act_i(x_i @ W_i) (+ residual_i)]`` as ONE launch of the decode GEMM, or ``None`` when the problems do not
    qualify (more than 128 rows, autograd recording, CPU tensors, odd shapes): the caller then takes its usual path.
    ``kn[i]`` marks a weight stored ``[in, out]``; ``acts[i]`` is ``None``, ``"relu_sq"``, ``"tanh"`` or ``"sigmoid"``."""
    n = _native()
    if not _decode(n) or torch.is_grad_enabled() or not 0 < len(xs) <= n.DECODE_MAX_PROBLEMS:
        return None
    kn = list(kn) if kn is not None else [False] * len(xs)
    x2 = [x.reshape(-1, x.shape[-1]) for x in xs]
    if any(a.shape[0] != x2[0].shape[0] for a in x2) or not all(n.decode_ok(a, w, t) for a, w, t in zip(x2, ws, kn)):
        return None
    r2 = None
    if residuals is not None:
        r2 = [None if r is None else r.reshape(-1, r.shape[-1]) for r in residuals]
        for r, w, t in zip(r2, ws, kn):
            if r is not None and not (r.dtype == torch.bfloat16 and r.is_contiguous() and r.data_ptr() % 8 == 0
                                      and r.shape == (x2[0].shape[0], w.shape[1] if t else w.shape[0])):
                return None
    ys = n.decode_group(x2, list(ws), epis=acts, kn=kn, residuals=r2, prefetch=prefetch)
    return [y.reshape(*x.shape[:-1], y.shape[-1]) for y, x in zip(ys, xs)]


def decode_projection_set(lin, lowrank=(), prefetch=None):
    """A set of independent projections of the same few rows, in at most two launches of the decode GEMM.
    ``prefetch``: weight tensors of the products that come next in the step (L2 prefetch hint, see ``decode_group``).

    ``lin``: ``(x, weight [out, in], act, residual, lora)`` per ``nn.Linear``-like map, ``lora`` being ``None`` or
    ``(A [r, in], B [out, r], scaling)``; the result is ``act(x W^T + scaling * (x A^T) B^T) + residual`` (a residual
    together with an activation is supported without an adapter only).  ``lowrank``: ``(x, w1 [in, d], act, w2 [d, out])``
    per chain, result ``act(x w1) w2``.  First launch: every base product, every ``x A^T`` and every chain's first stage;
    second launch: every adapter's ``B`` product accumulated in place (activation applied there) and every chain's second
    stage.  Returns ``(lin_outs, lowrank_outs)`` or ``None`` when the set does not qualify."""
    n = _native()
    if not _decode(n) or torch.is_grad_enabled():
        return None
    if any(lora is not None and act is not None and residual is not None for _, _, act, residual, lora in lin):
        return None
    adapters = [i for i, item in enumerate(lin) if item[4] is not None]
    # first launch, one row per problem: (x, weight, weight stored [in, out], activation, residual)
    first_rows = [(x, w, False, act if lora is None else None, residual if (lora is None or act is None) else None)
                  for x, w, act, residual, lora in lin]
    first_rows += [(lin[i][0], lin[i][4][0], False, None, None) for i in adapters]
    first_rows += [(x, w1, True, act, None) for x, w1, act, _ in lowrank]
    if not first_rows or len(first_rows) > n.DECODE_MAX_PROBLEMS:
        return None
    xs, ws, kn, acts, res = (list(col) for col in zip(*first_rows))
    first = decode_products(xs, ws, acts=acts, kn=kn, residuals=res, prefetch=prefetch)
    if first is None:
        return None
    n_lin = len(lin)
    lin_out = first[:n_lin]
    xa = first[n_lin:n_lin + len(adapters)]
    hidden = first[n_lin + len(adapters):]
    if not adapters and not lowrank:
        return lin_out, []
    # second launch: (x, weight, stored [in, out], activation, residual, scale, residual before activation, output)
    second_rows = []
    for a_out, i in zip(xa, adapters):
        y = lin_out[i].reshape(-1, lin_out[i].shape[-1])          # accumulated in place
        _, lora_b, scaling = lin[i][4]
        second_rows.append((a_out.reshape(-1, a_out.shape[-1]), lora_b, False, lin[i][2], y, scaling, True, y))
    for h, (_, _, _, w2) in zip(hidden, lowrank):
        second_rows.append((h.reshape(-1, h.shape[-1]), w2, True, None, None, 1.0, False, None))
    x2, w2s, kn2, act2, res2, alpha2, rf2, outs2 = (list(col) for col in zip(*second_rows))
    if not all(n.decode_ok(a, w, t) for a, w, t in zip(x2, w2s, kn2)):
        # the first launch has run; finish the set with ordinary products
        for a_out, i in zip(xa, adapters):
            _, lora_b, scaling = lin[i][4]
            y = lin_out[i] + (a_out @ lora_b.t()) * scaling
            lin_out[i] = y if lin[i][2] is None else _apply_act(y, lin[i][2])
        return lin_out, [h @ w2 for h, (_, _, _, w2) in zip(hidden, lowrank)]
    second = n.decode_group(x2, w2s, epis=act2, kn=kn2, residuals=res2, alphas=alpha2, res_first=rf2, outs=outs2)
    lows = [y.reshape(*item[0].shape[:-1], y.shape[-1]) for y, item in zip(second[len(adapters):], lowrank)]
    return lin_out, lows


def _apply_act(y: torch.Tensor, act: str) -> torch.Tensor:
    if act == "relu_sq":
        return torch.relu(y) ** 2
    return torch.tanh(y) if act == "tanh" else torch.sigmoid(y)


def mm_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    n = _native()
    if n is not None:
        if n.DECODE_DISPATCH and n.decode_ok(x, w):
            return n.decode_group([x], [w])[0]
        if n.native_ok(x, w, "nt"):
            return n.mm_nt(x, w)
    return x @ w.t()


def linear_group(xs, ws):
    """``[x_i @ w_i^T]`` for several independent projections with the same row count.  During decoding
    (few rows, no autograd) they go out as one grouped launch; otherwise one ``linear`` each."""
    ys = decode_products(xs, ws)
    if ys is not None:
        return ys
    return [linear(x, w) for x, w in zip(xs, ws)]


def projections_with_lowrank(lin_xs, lin_ws, lr_xs, lr_w1, lr_acts, lr_w2):
    """The projections of a time-mix block: ``[x @ W^T]`` for the ``nn.Linear`` weights ``lin_ws`` and
    ``[act(x @ w1) @ w2]`` for the low-rank chains.  While decoding (few rows, no autograd) the linear maps and all
    first stages are one grouped launch and all second stages another; otherwise one GEMM each."""
    out = decode_projection_set([(x, w, None, None, None) for x, w in zip(lin_xs, lin_ws)],
                                list(zip(lr_xs, lr_w1, lr_acts, lr_w2)))
    if out is not None:
        return out
    lins = [linear(x, w) for x, w in zip(lin_xs, lin_ws)]
    lows = [matmul(matmul_act(x, a, act) if act else matmul(x, a), b)
            for x, a, act, b in zip(lr_xs, lr_w1, lr_acts, lr_w2)]
    return lins, lows


def mm_nn(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    n = _native()
    if n is not None:
        if n.DECODE_DISPATCH and n.decode_ok(x, w, True):
            return n.decode_group([x], [w], kn=[True])[0]
        if n.native_ok(x, w, "nn"):
            return n.mm_nn(x, w)
    return x @ w


def _acc_ok(n, y: torch.Tensor) -> bool:
    return (n is not None and y.is_cuda and y.dtype == torch.bfloat16 and y.dim() == 2 and y.stride(1) == 1
            and y.data_ptr() % 16 == 0 and (y.stride(0) * 2) % 16 == 0)


def mm_nt_plus(x: torch.Tensor, w: torch.Tensor, x2: torch.Tensor, w2: torch.Tensor, act: str = None,
               residual: torch.Tensor = None) -> torch.Tensor:
    """``x @ w^T + x2 @ w2^T`` (``w [N, K]``, ``w2 [N, K2]``), optionally ``relu(.)^2`` (``act="relu_sq"``) or plus a
    ``residual [M, N]`` (not both).  On the native path ONE GEMM launch whose contraction runs over ``K`` then ``K2`` (the
    LoRA linear: ``x2 = s x A^T``, ``w2 = B``) with the activation / residual sum in its epilogue; otherwise a GEMM, an
    accumulate and a separate element-wise pass."""
    if act not in (None, "relu_sq") or (act is not None and residual is not None):
        raise ValueError("mm_nt_plus: act is None or 'relu_sq', and never together with a residual")
    n = _native()
    if n is not None and n.dual_ok(x, w, x2, w2, "nt") and (residual is None or _acc_ok(n, residual)):
        return n.mm_nt_dual(x, w, x2, w2, epilogue=1 if act else 0, residual=residual)
    y = addmm_nt_(mm_nt(x, w), x2, w2)
    if act:
        y = torch.relu(y) ** 2
    return y if residual is None else y + residual


def mm_nn_plus(x: torch.Tensor, w: torch.Tensor, x2: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """``x @ w + x2 @ w2`` (``w [K, N]``, ``w2 [K2, N]``); see :func:`mm_nt_plus`."""
    n = _native()
    if n is not None and n.dual_ok(x, w, x2, w2, "nn"):
        return n.mm_nn_dual(x, w, x2, w2)
    return addmm_nn_(mm_nn(x, w), x2, w2)


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
        if _decode(n) and n.decode_ok(x2, w) and r2.dtype == torch.bfloat16 and r2.is_contiguous():
            y = n.decode_group([x2], [w], residuals=[r2])[0]
        elif _acc_ok(n, r2) and n.native_ok(x2, w, "nt"):
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
        if _decode(n) and n.decode_ok(x2, w, True):
            y = n.decode_group([x2], [w], epis=[act], kn=[True])[0]
        elif n is not None and n.native_ok(x2, w, "nn"):
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
