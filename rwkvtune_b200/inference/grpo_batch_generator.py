"""Batched rollout generation for GRPO.

Same contract as ``rwkvtune/inference/grpo_batch_generator.py:115-351``: prompts are de-duplicated,
unique prompts are prefilled once (grouped by equal length, in chunks), the recurrent state is
copied to the ``G`` paths of each prompt, the first token is sampled from the prefill logits and all
paths then decode in lock-step until EOS (kept in the completion) or ``max_new_tokens``.  Returns
``{"completions", "completion_ids" [B*G, max_len] 0-padded, "masks" bool}``.

What differs is where the loop lives.  The reference syncs to the host for every sequence and token
(``.item()`` per token, Python repetition penalty, gather/scatter of per-sequence state dicts).  Here
the sampled ids, EOS detection, length counters and the repetition-penalty bitmap stay on the
device; the host looks at a single "all finished" flag every ``sync_every`` steps and compacts the
batch when more than half of the paths are done.
"""
from __future__ import annotations

import contextlib
import time
import weakref
from typing import Any, Dict, List, Optional, Sequence

import torch

from .. import ops
from ..ops import _ext as _ext_mod
from . import sampling_native
from .core import TokenSampler, apply_repetition_penalty


class _DecodeGraph:
    """One decode step (all layers + head) for a fixed number of sequences, captured as a CUDA graph.
    The recurrent state lives in static buffers that the captured step updates in place, so a replay
    costs one launch instead of several hundred."""

    def __init__(self, gen: "GRPOBatchGenerator", n: int):
        from ..ops import cuda_ops

        self.gen, self.n = weakref.proxy(gen), n      # no cycle generator <-> graph: both die by reference count
        dev = gen.device
        self.tok = torch.zeros(n, 1, dtype=torch.long, device=dev)
        self.state = gen._zero_state(n)
        cuda_ops.INPLACE_STATE = True
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._body()
            torch.cuda.current_stream(dev).wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with _ext_mod.capture_safe_gc(), torch.cuda.graph(self.graph):
                self.logits = self._body()
        finally:
            cuda_ops.INPLACE_STATE = False

    def _body(self) -> torch.Tensor:
        logits, (a, s, f) = self.gen._forward(self.tok, self.state)
        for dst, src in zip(self.state[0], a):
            dst.copy_(src)
        for dst, src in zip(self.state[1], s):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        for dst, src in zip(self.state[2], f):
            dst.copy_(src)
        return logits

    def load_state(self, state) -> None:
        for part_dst, part_src in zip(self.state, state):
            for dst, src in zip(part_dst, part_src):
                dst.copy_(src)

    def step(self, tok: Optional[torch.Tensor]) -> torch.Tensor:
        """Replay the captured step on ``tok``; ``None`` when the caller has already written ``self.tok``."""
        if tok is not None:
            self.tok.copy_(tok[:, None])
        self.graph.replay()
        return self.logits


class GRPOBatchGenerator:
    def __init__(self, model, tokenizer=None, device=None, eos_token_id=None, prefill_chunk_size: int = 2048,
                 max_prefill_batch_size: int = -1, max_decode_batch_size: int = -1, sync_every: int = 8,
                 verbose: bool = False, use_cuda_graph: Optional[bool] = None, chunk_size: Optional[int] = None):
        if chunk_size is not None:      # the reference's name for the prefill chunk (grpo_batch_generator.py:74-82)
            prefill_chunk_size = chunk_size
        self.model = model
        self.tokenizer = tokenizer
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        eos = eos_token_id
        if eos is None and tokenizer is not None:
            eos = getattr(tokenizer, "eos_token_id", None)
        if eos is None:
            eos = getattr(model.config, "eos_token_id", None)
        self.eos_ids = [] if eos is None else ([int(eos)] if isinstance(eos, int) else [int(e) for e in eos])
        self.prefill_chunk_size = self.chunk_size = prefill_chunk_size
        self.max_prefill_batch_size = max_prefill_batch_size
        self.max_decode_batch_size = max_decode_batch_size
        self.sync_every = max(1, sync_every)
        self.verbose = verbose
        self.max_valid_token_id = None
        if tokenizer is not None and hasattr(tokenizer, "vocab_size"):
            self.max_valid_token_id = int(tokenizer.vocab_size) - 1
        self.last_stats: Dict[str, float] = {}
        sharded = any(getattr(m, "_sharded", None) is not None for m in model.modules())
        self.use_cuda_graph = (self.device.type == "cuda" and not sharded) if use_cuda_graph is None else use_cuda_graph
        self._graphs: Dict[int, _DecodeGraph] = {}

    def _graph_for(self, n: int) -> "_DecodeGraph":
        if n not in self._graphs:
            if len(self._graphs) >= 6:
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[n] = _DecodeGraph(self, n)
        return self._graphs[n]

    # ------------------------------------------------------------------ state helpers
    def _zero_state(self, n: int):
        cfg, m = self.model.config, self.model
        H, N = cfg.dim_att // cfg.head_size_a, cfg.head_size_a
        L = cfg.n_layer
        att = [torch.zeros(n, cfg.n_embd, dtype=m.dtype, device=self.device) for _ in range(L)]
        wkv = [torch.zeros(n, H, N, N, dtype=torch.float32, device=self.device) for _ in range(L)]
        ffn = [torch.zeros(n, cfg.n_embd, dtype=m.dtype, device=self.device) for _ in range(L)]
        return att, wkv, ffn

    @staticmethod
    def _select(state, index: torch.Tensor):
        return tuple([ops.gather_rows(t, index) for t in part] for part in state)

    def _forward(self, ids: torch.Tensor, state):
        from ..ops import _ext

        att, wkv, ffn = state
        # weights are constant for the whole rollout: the step's kernels can be launched as a dependent chain
        with (_ext.launch_chaining() if ids.is_cuda and ids.shape[1] == 1 else contextlib.nullcontext()):
            x, a, s, f = self.model.forward_states(ids, att, wkv, ffn)
            logits = self.model.head(x[:, -1, :])
        return logits, (a, s, f)

    # ------------------------------------------------------------------ prefill
    def _chunked_prefill(self, prompts: List[List[int]]):
        """Prefill unique prompts; returns (last-position logits [U, V], state for the U prompts)."""
        U = len(prompts)
        state = self._zero_state(U)
        V = self.model.config.vocab_size
        logits_out = torch.empty(U, V, dtype=torch.float32, device=self.device)
        by_len: Dict[int, List[int]] = {}
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError("empty prompt")
            by_len.setdefault(len(p), []).append(i)
        cap = self.max_prefill_batch_size if self.max_prefill_batch_size and self.max_prefill_batch_size > 0 else U
        for length, members in by_len.items():
            for g0 in range(0, len(members), cap):
                grp = members[g0:g0 + cap]
                idx = torch.tensor(grp, dtype=torch.long, device=self.device)
                ids = torch.tensor([prompts[i] for i in grp], dtype=torch.long, device=self.device)
                st = self._select(state, idx)
                logits = None
                for c0 in range(0, length, self.prefill_chunk_size):
                    logits, st = self._forward(ids[:, c0:c0 + self.prefill_chunk_size], st)
                for part, new in zip(state, st):
                    for dst, src in zip(part, new):
                        dst.index_copy_(0, idx, src.to(dst.dtype))
                logits_out.index_copy_(0, idx, logits.float())
        return logits_out, state

    # ------------------------------------------------------------------ main entry
    @torch.no_grad()
    def generate(self, input_ids: Sequence[Sequence[int]], max_new_tokens: int = 256, num_generations: int = 1,
                 temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0, repetition_penalty: float = 1.0,
                 logit_bias: Optional[Dict[int, float]] = None, seed: Optional[int] = None,
                 return_text: bool = True) -> Dict[str, Any]:
        was_training = self.model.training
        self.model.eval()
        t_start = time.perf_counter()
        dev = self.device
        prompts = [list(map(int, p)) for p in input_ids]
        B, G = len(prompts), int(num_generations)
        n = B * G
        uniq: Dict[tuple, int] = {}
        owner = []
        for p in prompts:
            owner.append(uniq.setdefault(tuple(p), len(uniq)))
        uniq_prompts = [list(k) for k in uniq.keys()]
        nvtx = dev.type == "cuda"
        if nvtx:
            torch.cuda.nvtx.range_push("prefill")
        pre_logits, pre_state = self._chunked_prefill(uniq_prompts)
        if nvtx:
            torch.cuda.nvtx.range_pop()
            torch.cuda.nvtx.range_push("decode")
        t_prefill = time.perf_counter()
        fan = torch.tensor(owner, dtype=torch.long, device=dev).repeat_interleave(G)
        state = self._select(pre_state, fan)
        logits = pre_logits.index_select(0, fan)
        del pre_state, pre_logits

        V = self.model.config.vocab_size
        prev_max = TokenSampler._max_valid_token_id
        TokenSampler.set_max_valid_token_id(self.max_valid_token_id)
        use_pen = repetition_penalty is not None and repetition_penalty != 1.0 and repetition_penalty > 0
        seen = None
        if use_pen:
            seen = torch.zeros(n, V, dtype=torch.bool, device=dev)
            for row, o in enumerate(fan.tolist()):
                seen[row, torch.tensor(uniq_prompts[o], device=dev).clamp(0, V - 1)] = True
        eos = torch.tensor(self.eos_ids, dtype=torch.long, device=dev) if self.eos_ids else None
        out_ids = torch.zeros(n, max_new_tokens, dtype=torch.long, device=dev)
        lengths = torch.zeros(n, dtype=torch.long, device=dev)
        finished = torch.zeros(n, dtype=torch.bool, device=dev)
        rows = torch.arange(n, device=dev)          # original row of each live path
        steps = 0
        graph = None
        if self.use_cuda_graph:
            graph = self._graph_for(n)
            graph.load_state(state)
        try:
            fused_sampler = (dev.type == "cuda" and TokenSampler.use_native_kernel and sampling_native.full_available()
                             and V <= 65536)
            fused_advance = dev.type == "cuda" and sampling_native.advance_available()
            for step in range(max_new_tokens):
                step_seed = None if seed is None else int(seed) * 1000003 + step
                if fused_sampler:   # penalty, ban, temperature, bias, top-k, top-p, draw and bitmap update: one launch
                    tok, _ = sampling_native.sample_tokens(
                        logits, temperature, top_p, top_k, logit_bias, self.max_valid_token_id,
                        seen=seen if use_pen else None, seen_rows=rows if use_pen else None,
                        repetition_penalty=repetition_penalty if use_pen else 1.0, update_seen=use_pen, seed=step_seed)
                else:
                    lg = logits.float()
                    if use_pen:
                        lg = apply_repetition_penalty(lg, seen.index_select(0, rows), repetition_penalty)
                    tok, _ = TokenSampler.sample_batch(lg, temperature, top_p, top_k, logit_bias, seed=step_seed)
                if use_pen and not fused_sampler:
                    seen[rows, tok] = True
                fed = False
                if fused_advance:   # token store, length count, end-of-sequence check, next step's input: one launch
                    fed = graph is not None
                    sampling_native.rollout_advance(tok, rows, finished, out_ids, lengths, eos, step,
                                                    graph.tok if fed else None)
                else:
                    live = ~finished.index_select(0, rows)
                    out_ids[rows, step] = torch.where(live, tok, torch.zeros_like(tok))
                    lengths[rows] += live.long()
                    done_now = torch.zeros_like(live)
                    if eos is not None:
                        done_now = torch.isin(tok, eos)
                    done_now |= (step + 1) >= max_new_tokens
                    finished[rows] |= done_now & live | ~live
                steps = step + 1
                if steps == max_new_tokens:
                    break
                if steps % self.sync_every == 0:
                    fin_live = finished.index_select(0, rows)
                    n_done = int(fin_live.sum())
                    if n_done == rows.numel():
                        break
                    if n_done * 2 >= rows.numel():   # compact: drop finished paths from the decode batch
                        keep = (~fin_live).nonzero(as_tuple=True)[0]
                        rows = rows.index_select(0, keep)
                        state = self._select(graph.state if graph is not None else state, keep)
                        tok = tok.index_select(0, keep)
                        fed = False                  # another batch size: the next step's input buffer changes
                        if graph is not None:
                            graph = self._graph_for(int(keep.numel()))
                            graph.load_state(state)
                if graph is not None:
                    logits = graph.step(None if fed else tok)
                else:
                    logits, state = self._forward(tok[:, None], state)
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()
            TokenSampler.set_max_valid_token_id(prev_max)
            if was_training:
                self.model.train()
        max_len = int(lengths.max()) if n else 0          # host read: everything queued above has completed
        if dev.type == "cuda":
            from ..ops import gemm_native

            code = gemm_native.check_status(dev) if gemm_native.available() else 0
            if code:      # a bounded device-side wait of a GEMM ran out during the rollout: the tokens are not trustworthy
                raise RuntimeError(f"rollout aborted: a device-side wait expired inside a GEMM kernel (status {code})")
        comp = out_ids[:, :max_len]
        masks = torch.arange(max_len, device=dev)[None, :] < lengths[:, None]
        comp = comp * masks
        t_end = time.perf_counter()
        gen_tokens = int(lengths.sum())
        self.last_stats = {"prefill_s": t_prefill - t_start, "decode_s": t_end - t_prefill, "steps": steps,
                           "generated_tokens": gen_tokens, "unique_prompts": len(uniq_prompts),
                           "decode_tok_s": gen_tokens / max(t_end - t_prefill, 1e-9)}
        if self.verbose:
            print(f"[rollout] {len(uniq_prompts)} unique prompts, {n} paths, {gen_tokens} tokens, "
                  f"prefill {self.last_stats['prefill_s']:.3f}s decode {self.last_stats['decode_s']:.3f}s "
                  f"({self.last_stats['decode_tok_s']:.0f} tok/s)")
        texts: List[str] = []
        if return_text and self.tokenizer is not None:
            host, lens = comp.tolist(), lengths.tolist()
            for row, ln in zip(host, lens):
                try:
                    texts.append(self.tokenizer.decode(row[:ln]))
                except Exception:
                    texts.append("")
        return {"completions": texts, "completion_ids": comp, "masks": masks, "lengths": lengths}
