"""RWKV-7 ("x070") network built from fused operator calls.

The parameter tree and names are those of the reference
(``rwkvtune/models/rwkv7/model.py:34-654``) so a ``model.pth`` written by either
project loads in the other.  The forward pass is *not* the reference's chain of
~45 framework ops per layer: each block is eight fused operator calls
(``rwkvtune_b200.ops``) that map one-to-one onto sm_100a kernels on a GPU and
onto plain PyTorch on the CPU.  One code path serves the three modes the
reference implements separately: training from a zero state
(``model.py:435-466``), stateful inference (``:468-497``) and infinite-context
training with the state carried between chunks
(``rwkvtune/models/rwkv7/model_infctx.py:200-255``).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint as _checkpoint

from ... import ops
from ..generation_mixin import GenerationMixin


class Linear(nn.Linear):
    """Bias-free ``nn.Linear`` whose matmul goes through the framework GEMM."""

    def __init__(self, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__(in_features, out_features, bias=False, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # noqa: D401
        sw = getattr(self, "_sharded", None)
        if sw is not None:   # ZeRO-3: weight lives as K-panels across ranks, gathered inside the GEMM
            from ...parallel.zero3 import ag_linear

            return ag_linear(x, sw)
        return ops.linear(x, self.weight)


def _decode_spec(layer: nn.Module, x: torch.Tensor, act: Optional[str] = None, residual: Optional[torch.Tensor] = None):
    """Entry of :func:`ops.decode_projection_set` for a projection layer: a plain unsharded :class:`Linear`, or a wrapper
    that describes itself through ``decode_spec()`` (the LoRA layer: base weight + adapter factors).  ``None`` for
    anything else (ZeRO-3 panels, adapters with active dropout)."""
    if getattr(layer, "_sharded", None) is not None:
        return None
    if type(layer) is Linear:
        return (x, layer.weight, act, residual, None)
    describe = getattr(layer, "decode_spec", None)
    spec = describe() if describe is not None else None
    if spec is None:
        return None
    return (x, spec[0], act, residual, spec[1])


def _decoding(x: torch.Tensor) -> bool:
    """Few rows, no autograd, on the GPU: the grouped decode GEMM applies."""
    return x.is_cuda and not torch.is_grad_enabled() and x.numel() // x.shape[-1] <= 128


def _weights_of(*layers) -> list:
    """Weight tensors of projection layers, as an L2 prefetch hint for the decode GEMM (sharded or absent ones skipped)."""
    out = []
    for m in layers:
        w = getattr(m, "weight", None) if m is not None else None
        if isinstance(w, torch.Tensor) and w.is_cuda and w.numel() > 0:
            out.append(w)
    return out


def _project_add(layer: nn.Module, h: torch.Tensor, residual: torch.Tensor, prefetch=None) -> torch.Tensor:
    """``residual + layer(h)``; a plain, unsharded :class:`Linear` adds the residual in its GEMM epilogue.  ``prefetch``:
    weights that the step reads next (decode only)."""
    if _decoding(h):
        spec = _decode_spec(layer, h, None, residual)
        out = ops.decode_projection_set([spec], (), prefetch) if spec is not None else None
        if out is not None:
            return out[0][0]
    if type(layer) is Linear and getattr(layer, "_sharded", None) is None:
        return ops.linear_add(h, layer.weight, residual)
    if getattr(layer, "lora_A", None) is not None:      # adapter layer: the residual sum rides in its fused GEMM
        return layer(h, residual=residual)
    return residual + layer(h)


def _ortho(rows: int, cols: int, scale: float, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    gain = math.sqrt(rows / cols) if rows > cols else 1.0
    w = torch.empty(rows, cols)
    nn.init.orthogonal_(w, gain=gain * scale, generator=generator)
    return w


def _low_rank_width(cfg_value: int, coeff: float, C: int) -> int:
    if cfg_value and cfg_value > 0:
        return int(cfg_value)
    return max(32, int(round((coeff * (C ** 0.5)) / 32) * 32))


class RWKV7TimeMix(nn.Module):
    """Time-mix ("attention") half of a block; init formulas follow ``model.py:48-117``."""

    def __init__(self, config, layer_id: int):
        super().__init__()
        self.config = config
        self.layer_id = layer_id
        self.head_size = config.head_size_a
        C = config.n_embd
        self.n_head = H = config.dim_att // self.head_size
        N = self.head_size
        L = config.n_layer

        r01 = layer_id / max(L - 1, 1)
        r10 = 1.0 - layer_id / L
        idx = torch.arange(C, dtype=torch.float32)
        ddd = (idx / C).reshape(1, 1, C)
        linear = idx / max(C - 1, 1) - 0.5
        zz = ((idx % N) - (N - 1) / 2) / ((N - 1) / 2)
        zigzag = zz * zz.abs()
        www = -6 + 6 * (idx / max(C - 1, 1)) ** (1 + r01 ** 0.3)

        P = nn.Parameter
        self.x_r = P(1.0 - ddd.pow(0.2 * r10))
        self.x_w = P(1.0 - ddd.pow(0.9 * r10))
        self.x_k = P(1.0 - ddd.pow(0.7 * r10))
        self.x_v = P(1.0 - ddd.pow(0.7 * r10))
        self.x_a = P(1.0 - ddd.pow(0.9 * r10))
        self.x_g = P(1.0 - ddd.pow(0.2 * r10))

        Dw = _low_rank_width(getattr(config, "dim_att_lora", 0), 2.0, C)
        self.w1 = P(torch.zeros(C, Dw))
        self.w2 = P(_ortho(Dw, C, 0.1))
        self.w0 = P((www + 0.5 + zigzag * 2.5).reshape(1, 1, C))

        self.a1 = P(torch.zeros(C, Dw))
        self.a2 = P(_ortho(Dw, C, 0.1))
        self.a0 = P((-0.19 + zigzag * 0.3 + linear * 0.4).reshape(1, 1, C))

        if layer_id > 0:
            Dv = _low_rank_width(getattr(config, "dim_mv_lora", 0), 1.4, C)
            self.v1 = P(torch.zeros(C, Dv))
            self.v2 = P(_ortho(Dv, C, 0.1))
            self.v0 = P((0.73 - linear * 0.4).reshape(1, 1, C))

        Dg = _low_rank_width(getattr(config, "dim_gate_lora", 0), 5.6, C)
        self.g1 = P(torch.zeros(C, Dg))
        self.g2 = P(_ortho(Dg, C, 0.1))

        self.k_k = P((0.71 - linear * 0.1).reshape(1, 1, C))
        self.k_a = P(torch.full((1, 1, C), 1.02))
        self.r_k = P(torch.full((H, N), -0.04))

        self.receptance = Linear(C, C)
        self.key = Linear(C, C)
        self.value = Linear(C, C)
        self.output = Linear(C, C)
        self.ln_x = nn.GroupNorm(H, C, eps=ops.GROUPNORM_EPS)
        with torch.no_grad():
            s = C ** -0.5
            self.receptance.weight.uniform_(-0.5 * s, 0.5 * s)
            self.key.weight.uniform_(-0.05 * s, 0.05 * s)
            self.value.weight.uniform_(-0.5 * s, 0.5 * s)
            self.output.weight.zero_()

    def _plain_projections(self) -> bool:
        """True when r/k/v are unwrapped, unsharded ``Linear`` layers (no adapter, no ZeRO-3 panels)."""
        return all(type(m) is Linear and getattr(m, "_sharded", None) is None
                   for m in (self.receptance, self.key, self.value))

    def mix_matrix(self) -> torch.Tensor:
        C = self.x_r.shape[-1]
        if not torch.is_grad_enabled():   # inference: one cached [6, C] parameter-like tensor, rebuilt when weights change
            key = tuple(p._version for p in (self.x_r, self.x_w, self.x_k, self.x_v, self.x_a, self.x_g)) + (ops.param_epoch(),)
            cached = getattr(self, "_mix_cache", None)
            if cached is None or cached[0] != key or cached[1].device != self.x_r.device:
                m = torch.cat([self.x_r, self.x_w, self.x_k, self.x_v, self.x_a, self.x_g], dim=0).reshape(6, C)
                cached = (key, torch.nn.Parameter(m.detach().clone(), requires_grad=False))
                object.__setattr__(self, "_mix_cache", cached)
            return cached[1]
        return torch.cat([self.x_r, self.x_w, self.x_k, self.x_v, self.x_a, self.x_g], dim=0).reshape(6, C)

    def forward(self, x, ln_w, ln_b, v_first, x_prev=None, wkv_state=None, want_state: bool = False):
        """``x`` is the *pre-LayerNorm* residual stream ``[B, T, C]``.

        Returns ``(x + out, v_first, last_ln_row, new_wkv_state)`` - the updated residual stream, not the
        bare projection; the last two are ``None`` unless ``want_state``.
        """
        (xr, xw, xk, xv, xa, xg), last, x = ops.ln_shift_mix_unbound(x, ln_w, ln_b, self.mix_matrix(), x_prev)

        v_lin = None
        first = self.layer_id == 0
        done = False
        if x.is_cuda and not torch.is_grad_enabled():
            # inference: r/k/v (with their adapters, if any) and the first stages of the low-rank chains go out as one
            # grouped launch while decoding, the second stages as another
            chains = [(xw, self.w1, "tanh", self.w2), (xa, self.a1, None, self.a2), (xg, self.g1, "sigmoid", self.g2)]
            if not first:
                chains.append((xv, self.v1, None, self.v2))
            specs = [_decode_spec(m, t) for m, t in ((self.receptance, xr), (self.key, xk), (self.value, xv))]
            out = None
            if _decoding(x) and all(sp is not None for sp in specs):
                out = ops.decode_projection_set(specs, chains, _weights_of(self.output))
            if out is not None:
                (r, k, v), low = out
            elif self._plain_projections():
                (r, k, v), low = ops.projections_with_lowrank(
                    [xr, xk, xv], [self.receptance.weight, self.key.weight, self.value.weight],
                    [c[0] for c in chains], [c[1] for c in chains], [c[2] for c in chains], [c[3] for c in chains])
            else:
                r, k, v = self.receptance(xr), self.key(xk), self.value(xv)
                _, low = ops.projections_with_lowrank([], [], [c[0] for c in chains], [c[1] for c in chains],
                                                      [c[2] for c in chains], [c[3] for c in chains])
            w_lin, a_lin, g = low[:3]
            if not first:
                v_lin = low[3]
            done = True
        if not done:
            r = self.receptance(xr)
            k = self.key(xk)
            v = self.value(xv)
            w_lin = ops.matmul(ops.matmul_act(xw, self.w1, "tanh"), self.w2)
            a_lin = ops.matmul(ops.matmul(xa, self.a1), self.a2)
            g = ops.matmul(ops.matmul_act(xg, self.g1, "sigmoid"), self.g2)
            if not first:
                v_lin = ops.matmul(ops.matmul(xv, self.v1), self.v2)
        if ops.timemix_decode_core_ok(r, g, wkv_state, self.head_size):
            # one token per sequence: preparation, state update and GroupNorm + bonus + gate are one kernel
            z, new_state = ops.timemix_decode_core(r, k, v, None if first else v_first, w_lin, a_lin, v_lin, g, self.w0,
                                                   self.a0, None if first else self.v0, self.k_k, self.k_a, self.r_k,
                                                   self.ln_x.weight, self.ln_x.bias, wkv_state)
            if first:
                v_first = v
            nxt = getattr(self, "_decode_next", None)          # the channel-mix half of this block
            out = _project_add(self.output, z, x, _weights_of(getattr(nxt, "key", None)))
            return out, v_first, (last if want_state else None), (new_state if want_state else None)
        if self.layer_id == 0:
            w, k, v, a_, b_ = ops.timemix_prep(k, v, None, w_lin, a_lin, None, self.w0, self.a0, None,
                                               self.k_k, self.k_a, self.head_size)
            v_first = v
        else:
            w, k, v, a_, b_ = ops.timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, self.w0, self.a0, self.v0,
                                               self.k_k, self.k_a, self.head_size)

        # wkv_state may be (state pool [n_slots, H, N, N], slot index per sequence): updated in place by the kernel
        z, new_state = ops.wkv7_gn(r, w, k, v, a_, b_, g, self.ln_x.weight, self.ln_x.bias, self.r_k, self.head_size,
                                   state=wkv_state, return_state=want_state)
        out = _project_add(self.output, z, x)      # x + output(z): the residual sum rides in the GEMM epilogue
        return out, v_first, (last if want_state else None), new_state


    def forward_with_state(self, x, v_first, x_prev, att_kv):
        """The half-block step with the reference's module-level contract (``model.py:174-278``): ``x`` is the
        *normalised* input ``[B, T, C]``, ``x_prev`` the last normalised row of the previous call ``[B, C]``,
        ``att_kv`` the state ``[B, H, N, N]``.  Returns the bare projection ``(y, v_first, new_x_prev fp32,
        new_att_kv)`` - no residual sum.  A composition of the unfused ops for callers that drive the halves
        themselves; the model's own paths go through :meth:`forward`."""
        from ...ops import reference as _ref

        xx = _ref.token_shift(x, x_prev) - x
        xr, xw, xk, xv, xa, xg = (x + xx * m for m in (self.x_r, self.x_w, self.x_k, self.x_v, self.x_a, self.x_g))
        r, k, v = self.receptance(xr), self.key(xk), self.value(xv)
        w_lin = ops.matmul(ops.matmul_act(xw, self.w1, "tanh"), self.w2)
        a_lin = ops.matmul(ops.matmul(xa, self.a1), self.a2)
        g = ops.matmul(ops.matmul_act(xg, self.g1, "sigmoid"), self.g2)
        if self.layer_id == 0:
            w, k, v, a_, b_ = ops.timemix_prep(k, v, None, w_lin, a_lin, None, self.w0, self.a0, None, self.k_k, self.k_a,
                                               self.head_size)
            v_first = v
        else:
            v_lin = ops.matmul(ops.matmul(xv, self.v1), self.v2)
            w, k, v, a_, b_ = ops.timemix_prep(k, v, v_first, w_lin, a_lin, v_lin, self.w0, self.a0, self.v0, self.k_k,
                                               self.k_a, self.head_size)
        z, new_state = ops.wkv7_gn(r, w, k, v, a_, b_, g, self.ln_x.weight, self.ln_x.bias, self.r_k, self.head_size,
                                   state=att_kv.float(), return_state=True)
        return self.output(z), v_first, x[:, -1].float(), new_state


class RWKV7ChannelMix(nn.Module):
    """Squared-ReLU feed-forward half of a block (``model.py:281-343``); width is ``4 * n_embd``."""

    def __init__(self, config, layer_id: int):
        super().__init__()
        self.config = config
        self.layer_id = layer_id
        C = config.n_embd
        r10 = 1.0 - layer_id / config.n_layer
        ddd = (torch.arange(C, dtype=torch.float32) / C).reshape(1, 1, C)
        self.x_k = nn.Parameter(1.0 - ddd.pow(r10 ** 4))
        self.key = Linear(C, 4 * C)
        self.value = Linear(4 * C, C)
        with torch.no_grad():
            s = C ** -0.5
            self.key.weight.uniform_(-0.5 * s, 0.5 * s)
            self.value.weight.zero_()

    def forward(self, x, ln_w, ln_b, x_prev=None, want_state: bool = False):
        (xk,), last, x = ops.ln_shift_mix_unbound(x, ln_w, ln_b, self.x_k, x_prev)
        if _decoding(xk):
            spec = _decode_spec(self.key, xk, "relu_sq")
            out = ops.decode_projection_set([spec], (), _weights_of(self.value)) if spec is not None else None
            if out is not None:
                nxt = getattr(self, "_decode_next", None)      # the time-mix half of the next block
                hint = _weights_of(*(getattr(nxt, n, None) for n in ("receptance", "key", "value"))) if nxt is not None else None
                return _project_add(self.value, out[0][0], x, hint), (last if want_state else None)
        plain = all(type(m) is Linear and getattr(m, "_sharded", None) is None for m in (self.key, self.value))
        if plain:
            return ops.channel_mix_ffn(xk, self.key.weight, self.value.weight, x), (last if want_state else None)
        if type(self.key) is Linear and getattr(self.key, "_sharded", None) is None:
            hidden = ops.linear_relu_sq(xk, self.key.weight)
        elif getattr(self.key, "lora_A", None) is not None:     # adapter layer: relu^2 in the epilogue of its fused GEMM
            hidden = self.key(xk, act="relu_sq")
        else:   # sharded (ZeRO-3): activation applied separately
            hidden = ops.relu_squared(self.key(xk))
        return _project_add(self.value, hidden, x), (last if want_state else None)


    def forward_with_state(self, x, x_prev):
        """Reference contract of the half-block step (``model.py:310-343``): ``x`` normalised ``[B, T, C]``, ``x_prev``
        ``[B, C]``; returns ``(y, new_x_prev fp32)`` without the residual sum."""
        from ...ops import reference as _ref

        xk = x + (_ref.token_shift(x, x_prev) - x) * self.x_k
        return self.value(ops.relu_squared(self.key(xk))), x[:, -1].float()


class RWKV7Block(nn.Module):
    def __init__(self, config, layer_id: int):
        super().__init__()
        self.config = config
        self.layer_id = layer_id
        self.ln1 = nn.LayerNorm(config.n_embd)
        self.ln2 = nn.LayerNorm(config.n_embd)
        self.skip_ln0 = False
        if layer_id == 0:
            self.ln0 = nn.LayerNorm(config.n_embd)
        self.att = RWKV7TimeMix(config, layer_id)
        self.ffn = RWKV7ChannelMix(config, layer_id)

    def forward(self, x, v_first, att_prev=None, wkv_state=None, ffn_prev=None, want_state: bool = False):
        if self.layer_id == 0 and not self.skip_ln0:
            x = ops.layer_norm(x, self.ln0.weight, self.ln0.bias)
        # both halves return the updated residual stream
        x, v_first, att_last, new_wkv = self.att(x, self.ln1.weight, self.ln1.bias, v_first,
                                                 att_prev, wkv_state, want_state)
        x, ffn_last = self.ffn(x, self.ln2.weight, self.ln2.bias, ffn_prev, want_state)
        return x, v_first, att_last, new_wkv, ffn_last

    def forward_with_state(self, x, v_first, layer_state: Dict[str, torch.Tensor]):
        """Dictionary form of the stateful step (``rwkvtune/models/rwkv7/model.py:382-420``): ``layer_state`` holds
        ``att_x_prev`` / ``att_kv`` / ``ffn_x_prev``; returns ``(x, v_first, new_layer_state)`` with fp32 states."""
        dt = x.dtype
        x, v_first, att_last, new_wkv, ffn_last = self.forward(
            x, v_first, layer_state["att_x_prev"].to(dt), layer_state["att_kv"].float(),
            layer_state["ffn_x_prev"].to(dt), True)
        return x, v_first, {"att_x_prev": att_last.float(), "att_kv": new_wkv.float(), "ffn_x_prev": ffn_last.float()}


def _block_plain(block, x, v_first):
    x, v_first, _, _, _ = block(x, v_first)
    return x, v_first


def _block_stateful(block, x, v_first, att_prev, wkv_state, ffn_prev):
    return block(x, v_first, att_prev, wkv_state, ffn_prev, True)


class _Recompute(torch.autograd.Function):
    """Activation checkpointing of one block: run it without a graph, keep only its inputs, run it again with a
    graph when the gradient arrives.  Does what ``torch.utils.checkpoint`` does for this model
    (``rwkvtune/models/rwkv7/model.py:454-455`` wraps every block) without the per-saved-tensor pack/unpack hooks of
    the non-reentrant implementation, which cost more host time than the kernels of a small block.  ``anchor`` is an
    empty tensor that requires grad, so the node is part of the graph even when no real input requires grad (frozen
    embedding under LoRA); parameter gradients accumulate into ``.grad`` during the inner backward."""

    @staticmethod
    def forward(ctx, fn, block, anchor, *tensors):
        ctx.fn, ctx.block = fn, block
        ctx.req = [t is not None and t.requires_grad for t in tensors]
        ctx.none = [t is None for t in tensors]
        ctx.save_for_backward(*[t for t in tensors if t is not None])
        with torch.no_grad():
            outs = fn(block, *tensors)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        saved = iter(ctx.saved_tensors)
        inputs = [None if is_none else next(saved).detach().requires_grad_(req)
                  for is_none, req in zip(ctx.none, ctx.req)]
        with torch.enable_grad():
            outs = ctx.fn(ctx.block, *inputs)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None, None) + tuple(t.grad if t is not None and t.requires_grad else None for t in inputs)


def _has_active_dropout(block: nn.Module) -> bool:
    return block.training and any(isinstance(m, nn.Dropout) and m.p > 0 for m in block.modules())


def _checkpoint_block(fn, block, *tensors):
    """Recompute-in-backward wrapper for one block (random-number state is only preserved by the library path)."""
    if _has_active_dropout(block):
        return _checkpoint(fn, block, *tensors, use_reentrant=False)
    anchor = torch.empty(0, device=tensors[0].device, requires_grad=True)
    return _Recompute.apply(fn, block, anchor, *tensors)


class RWKV7Model(GenerationMixin, nn.Module):
    """Full model: embedding, ``n_layer`` blocks, final LayerNorm and the vocabulary head."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.emb = nn.Embedding(config.vocab_size, config.n_embd)
        self.blocks = nn.ModuleList([RWKV7Block(config, i) for i in range(config.n_layer)])
        # who runs after whom in a decode step (plain attributes, not sub-modules): each half tells its last GEMM whose
        # weights to bring into L2 next
        for i, blk in enumerate(self.blocks):
            object.__setattr__(blk.att, "_decode_next", blk.ffn)
            object.__setattr__(blk.ffn, "_decode_next", self.blocks[i + 1].att if i + 1 < config.n_layer else None)
        self.ln_out = nn.LayerNorm(config.n_embd)
        self.head = Linear(config.n_embd, config.vocab_size)
        self._emb_preprocessed = False

    # ------------------------------------------------------------------ helpers
    @property
    def device(self) -> torch.device:
        return self.emb.weight.device

    @property
    def dtype(self) -> torch.dtype:
        return self.emb.weight.dtype

    def _use_checkpoint(self) -> bool:
        return bool(getattr(self.config, "grad_cp", 0) == 1 and self.training and torch.is_grad_enabled())

    # ------------------------------------------------------------------ hidden states
    def forward_hidden(self, idx: torch.Tensor) -> torch.Tensor:
        """Run embedding and all blocks from a zero state; returns ``ln_out`` output ``[B, T, C]``."""
        B, T = idx.shape
        if T > self.config.ctx_len:
            raise ValueError(f"sequence length {T} exceeds ctx_len {self.config.ctx_len}")
        x = ops.embedding(idx, self.emb.weight)
        v_first = torch.empty_like(x)
        cp = self._use_checkpoint()
        n_cp = getattr(self.config, "grad_cp_layers", None)   # None: every layer; k: only the first k layers
        for i, block in enumerate(self.blocks):
            if cp and (n_cp is None or i < n_cp):
                x, v_first = _checkpoint_block(_block_plain, block, x, v_first)
            else:
                x, v_first = _block_plain(block, x, v_first)
        return ops.layer_norm(x, self.ln_out.weight, self.ln_out.bias)

    def forward(self, idx: torch.Tensor, logits_to_keep: Optional[int] = None) -> torch.Tensor:
        """Logits ``[B, T, V]`` (or the last ``logits_to_keep`` positions), ``model.py:435-466``."""
        x = self.forward_hidden(idx)
        if logits_to_keep is not None and logits_to_keep < x.shape[1]:
            x = x[:, -logits_to_keep:, :]
        return self.head(x)

    def loss(self, idx: torch.Tensor, labels: torch.Tensor, l2wrap: bool = True) -> torch.Tensor:
        """Mean cross-entropy over targets ``!= -100`` plus L2Wrap, without materialising the logits.

        Equivalent to ``CrossEntropyLoss(ignore_index=-100)(model(idx).view(-1, V), labels.view(-1))``
        followed by ``L2Wrap`` (``rwkvtune/training/lightning_module.py:175-206``).
        """
        x = self.forward_hidden(idx)
        B, T, C = x.shape
        return ops.linear_cross_entropy(x.reshape(B * T, C), self._head_weight(), labels.reshape(-1),
                                        l2wrap=l2wrap, l2wrap_tokens=B * T)

    def _head_weight(self) -> torch.Tensor:
        head = self.head
        if hasattr(head, "base_layer"):  # LoRA-wrapped heads are merged on the fly
            return head.effective_weight()
        return head.weight

    # ------------------------------------------------------------------ stateful paths
    def init_state(self, batch_size: int) -> List[Dict[str, torch.Tensor]]:
        """One dict per layer: ``att_x_prev [B,C]``, ``att_kv [B,H,N,N]`` fp32, ``ffn_x_prev [B,C]``."""
        cfg = self.config
        H, N = cfg.dim_att // cfg.head_size_a, cfg.head_size_a
        dev, dt = self.device, self.dtype
        return [
            {
                "att_x_prev": torch.zeros(batch_size, cfg.n_embd, dtype=dt, device=dev),
                "att_kv": torch.zeros(batch_size, H, N, N, dtype=torch.float32, device=dev),
                "ffn_x_prev": torch.zeros(batch_size, cfg.n_embd, dtype=dt, device=dev),
            }
            for _ in range(cfg.n_layer)
        ]

    def forward_states(self, idx, att_prev: Sequence[torch.Tensor], wkv: Sequence[torch.Tensor],
                       ffn_prev: Sequence[torch.Tensor], checkpoint: bool = False):
        """Blocks with state in and out.  Returns ``(hidden, att_last[L], wkv[L], ffn_last[L])``.

        Gradients flow through the incoming states, which is what full
        back-propagation through time across chunks needs.
        """
        x = ops.embedding(idx, self.emb.weight)
        v_first = torch.empty_like(x)
        new_att, new_wkv, new_ffn = [], [], []
        for i, block in enumerate(self.blocks):
            if checkpoint:
                x, v_first, a_l, s_l, f_l = _checkpoint_block(_block_stateful, block, x, v_first, att_prev[i], wkv[i],
                                                              ffn_prev[i])
            else:
                x, v_first, a_l, s_l, f_l = _block_stateful(block, x, v_first, att_prev[i], wkv[i], ffn_prev[i])
            new_att.append(a_l)
            new_wkv.append(s_l)
            new_ffn.append(f_l)
        x = ops.layer_norm(x, self.ln_out.weight, self.ln_out.bias)
        return x, new_att, new_wkv, new_ffn

    def forward_with_state(self, idx: torch.Tensor, states: Optional[List[Dict[str, torch.Tensor]]] = None,
                           last_only: bool = False):
        """Stateful inference step (prefill chunk or decode); ``model.py:468-497``.

        Returns ``(logits, new_states)``.  ``logits`` covers every position unless
        ``last_only`` (then ``[B, 1, V]``).  Carried rows are the post-LayerNorm
        activations of the last token, stored in fp32 like the reference does.
        """
        B, T = idx.shape
        if states is None:
            states = self.init_state(B)
        x, a_l, s_l, f_l = self.forward_states(
            idx, [s["att_x_prev"] for s in states], [s["att_kv"] for s in states],
            [s["ffn_x_prev"] for s in states])
        if last_only:
            x = x[:, -1:, :]
        logits = self.head(x)
        new_states = [
            {"att_x_prev": a.float(), "att_kv": s.float(), "ffn_x_prev": f.float()}
            for a, s, f in zip(a_l, s_l, f_l)
        ]
        return logits, new_states

    def forward_batch_dynamic(self, tokens_list: List[List[int]], states=None, full_output: bool = False):
        """Ragged batch forward (``model.py:522-585``): sequences advance in lock-step by the
        shortest remaining length until all are consumed."""
        n = len(tokens_list)
        lengths = [len(t) for t in tokens_list]
        if states is None:
            states = self.init_state(n)
        pos = [0] * n
        outs: List[Any] = [[] for _ in range(n)] if full_output else [None] * n
        while True:
            active = [i for i in range(n) if pos[i] < lengths[i]]
            if not active:
                break
            step = min(lengths[i] - pos[i] for i in active)
            ids = torch.tensor([tokens_list[i][pos[i]:pos[i] + step] for i in active], dtype=torch.long,
                               device=self.device)
            sub = [{k: v[active] for k, v in layer.items()} for layer in states]
            logits, new_sub = self.forward_with_state(ids, sub)
            for j, i in enumerate(active):
                if full_output:
                    outs[i].append(logits[j])
                else:
                    outs[i] = logits[j, -1]
                pos[i] += step
            for layer, new_layer in zip(states, new_sub):
                for key in layer:
                    layer[key][active] = new_layer[key].to(layer[key].dtype)
        if full_output:
            V = self.config.vocab_size
            outs = [torch.cat(o, dim=0) if o else torch.empty(0, V, dtype=self.dtype, device=self.device) for o in outs]
        return outs, states

    # ------------------------------------------------------------------ checkpoints
    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        """Accepts official RWKV-LM checkpoints (``model.py:607-654``): flat ``r_k`` is reshaped,
        layer-0 ``v0/v1/v2`` are dropped, the load is never strict, and a checkpoint without
        ``blocks.0.ln0.*`` marks the embedding as already normalised (``ln0`` is then skipped)."""
        sd = dict(state_dict)
        if "model" in sd and isinstance(sd["model"], dict) and "emb.weight" not in sd:
            sd = dict(sd["model"])
        has_ln0 = "blocks.0.ln0.weight" in sd and "blocks.0.ln0.bias" in sd
        H, N = self.config.dim_att // self.config.head_size_a, self.config.head_size_a
        for key in list(sd.keys()):
            if key.endswith("att.r_k") and sd[key].ndim == 1:
                sd[key] = sd[key].reshape(H, N)
        if len(self.blocks) and not hasattr(self.blocks[0].att, "v1"):
            for sfx in ("0", "1", "2"):
                sd.pop(f"blocks.0.att.v{sfx}", None)
        result = super().load_state_dict(sd, strict=False, assign=assign)
        self._emb_preprocessed = not has_ln0
        if len(self.blocks):
            self.blocks[0].skip_ln0 = not has_ln0
        return result

    def num_parameters(self, trainable_only: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)
