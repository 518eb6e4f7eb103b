"""Continuous-batching scheduler over a slot-indexed state pool.

Parity with ``rwkvtune/inference/scheduler_core.py:38-815``: sequences wait, prefill in chunks under a
token budget, then decode; decode always runs first; a finished sequence frees its slot for the next
waiting one; an optional :class:`StateCache` is consulted on admission; ``step_sync`` retries after a
CUDA out-of-memory error; ``run_to_completion_sync`` has a step cap and a no-progress watchdog.

The pool is three stacked tensors ``[L, max_batch, ...]`` (time-mix carried row, WKV state in fp32,
channel-mix carried row).  A step gathers the slots it works on with one ``index_select`` per tensor
and writes them back with one ``index_copy_``; the reference copies per sequence and per layer.
"""
from __future__ import annotations

import collections
import contextlib
import os
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Iterator, List, Optional, Tuple, Union

import torch

from ..ops import _ext
from .core import TokenSampler


def log_memory(tag: str) -> None:
    if os.environ.get("RWKV_DEBUG_MEMORY") == "1" and torch.cuda.is_available():
        print(f"[memory] {tag}: allocated {torch.cuda.memory_allocated() / 2**30:.2f} GB, "
              f"reserved {torch.cuda.memory_reserved() / 2**30:.2f} GB")


class SeqStatus(Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class SequenceState:
    seq_id: Union[int, str]
    prompt_tokens: List[int]
    status: SeqStatus = SeqStatus.WAITING
    prefill_offset: int = 0
    generated_tokens: List[int] = field(default_factory=list)
    last_token_id: Optional[int] = None
    max_new_tokens: int = 256
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    logit_bias: Optional[dict] = None
    stop: List[str] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    generated_text: str = ""
    slot_id: int = -1
    original_tokens: Optional[List[int]] = None
    cached_prefix_len: int = 0
    cached_state: Optional[Any] = None
    cached_output: Optional[torch.Tensor] = None
    output_queue: Optional[Any] = None
    enforcer: Optional[Any] = None
    enforcer_finished: bool = False
    finish_reason: Optional[str] = None
    pending_logits: Optional[torch.Tensor] = None

    @property
    def is_finished(self) -> bool:
        return self.status == SeqStatus.FINISHED

    @property
    def num_generated(self) -> int:
        return len(self.generated_tokens)


class SchedulerCore:
    def __init__(self, model, tokenizer, max_batch_size: int = 64, max_batch_tokens: int = 8192,
                 prefill_chunk_size: int = 512, state_cache=None):
        self.model, self.tokenizer = model, tokenizer
        self.device = next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        self.max_batch_size, self.max_batch_tokens = max_batch_size, max_batch_tokens
        self.prefill_chunk_size = prefill_chunk_size
        self.state_cache = state_cache
        cfg = model.config
        self.n_layer, self.n_embd = cfg.n_layer, cfg.n_embd
        self.head_size = getattr(cfg, "head_size_a", 64)
        self.n_head = cfg.dim_att // self.head_size
        self.state_pool = self._init_state_pool()
        self.sampler = TokenSampler
        if tokenizer is not None and getattr(tokenizer, "idx2token", None):
            TokenSampler.set_max_valid_token_id(max(tokenizer.idx2token.keys()))
        self.reset()

    def _init_state_pool(self) -> Dict[str, torch.Tensor]:
        L, n, C, H, N = self.n_layer, self.max_batch_size, self.n_embd, self.n_head, self.head_size
        log_memory("before state pool")
        pool = {"att_x_prev": torch.zeros(L, n, C, dtype=self.dtype, device=self.device),
                "att_kv": torch.zeros(L, n, H, N, N, dtype=torch.float32, device=self.device),
                "ffn_x_prev": torch.zeros(L, n, C, dtype=self.dtype, device=self.device)}
        log_memory("after state pool")
        return pool

    def reset(self) -> None:
        self.slots: List[Optional[SequenceState]] = [None] * self.max_batch_size
        self.free_slots = collections.deque(range(self.max_batch_size))
        self.waiting_queue: collections.deque = collections.deque()
        self.prefilling_seqs: List[SequenceState] = []
        self.running_seqs: List[SequenceState] = []
        self.finished_count = 0
        self.stop_reasons: Dict[str, int] = collections.Counter()
        for t in self.state_pool.values():
            t.zero_()

    # ------------------------------------------------------------------ queueing
    def add_sequences(self, sequences: List[SequenceState]) -> None:
        for s in sequences:
            self.add_sequence(s)

    def add_sequence(self, seq: SequenceState) -> None:
        if not seq.prompt_tokens:
            raise ValueError("a sequence needs at least one prompt token")
        seq.status = SeqStatus.WAITING
        self.waiting_queue.append(seq)

    def has_pending_work(self) -> bool:
        return bool(self.waiting_queue or self.prefilling_seqs or self.running_seqs)

    def get_stats(self) -> Dict[str, int]:
        return {"waiting": len(self.waiting_queue), "prefilling": len(self.prefilling_seqs),
                "running": len(self.running_seqs), "finished": self.finished_count, "free_slots": len(self.free_slots)}

    # ------------------------------------------------------------------ slots and state
    def _init_slot_state(self, seq: SequenceState, slot: int) -> None:
        self._reset_slot_state(slot)
        if self.state_cache is not None and self.state_cache.is_enabled():
            pos, state, out = self.state_cache.lookup(seq.prompt_tokens)
            if state is not None and pos > 0:
                self._load_state_to_slot(slot, state)
                seq.cached_prefix_len, seq.prefill_offset = pos, pos
                if pos == len(seq.prompt_tokens):
                    seq.pending_logits = out.float()

    def _reset_slot_state(self, slot: int) -> None:
        for t in self.state_pool.values():
            t[:, slot].zero_()

    def _load_state_to_slot(self, slot: int, state: List[Dict[str, torch.Tensor]]) -> None:
        for l, layer in enumerate(state):
            for k, pool in self.state_pool.items():
                pool[l, slot].copy_(layer[k].reshape(pool[l, slot].shape).to(pool.dtype))

    def _back_state_from_slot(self, slot: int) -> List[Dict[str, torch.Tensor]]:
        return [{k: pool[l, slot:slot + 1].float().clone() for k, pool in self.state_pool.items()}
                for l in range(self.n_layer)]

    @torch.no_grad()
    def _model_forward_with_state(self, ids: torch.Tensor, slots: List[int]) -> torch.Tensor:
        """One model call on the sequences in ``slots``.  The WKV states (16 KB per head and layer, by far the largest
        part of a sequence's state) are never gathered or scattered: the kernel reads and writes ``pool[slot]`` in
        place.  The two token-shift rows per layer go through ``index_select`` / ``index_copy_``."""
        idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        att = self.state_pool["att_x_prev"].index_select(1, idx)
        ffn = self.state_pool["ffn_x_prev"].index_select(1, idx)
        kv_pool = self.state_pool["att_kv"]
        if kv_pool.dtype == torch.float32 and kv_pool.is_contiguous():
            wkv = [(kv_pool[l], idx) for l in range(self.n_layer)]
        else:
            wkv = list(kv_pool.index_select(1, idx).unbind(0))
        # single-token steps of a serving loop (weights constant): the kernels are launched as a dependent chain
        chain = _ext.launch_chaining() if (ids.is_cuda and ids.shape[1] == 1) else contextlib.nullcontext()
        with chain:
            x, a, s, f = self.model.forward_states(ids, list(att.unbind(0)), wkv, list(ffn.unbind(0)))
        self.state_pool["att_x_prev"].index_copy_(1, idx, torch.stack(a).to(self.dtype))
        self.state_pool["ffn_x_prev"].index_copy_(1, idx, torch.stack(f).to(self.dtype))
        if not isinstance(s[0], tuple):
            kv_pool.index_copy_(1, idx, torch.stack(s).to(kv_pool.dtype))
        return self.model.head(x[:, -1, :]).float()

    def _finish_sequence(self, seq: SequenceState, reason: str) -> None:
        seq.status, seq.finish_reason = SeqStatus.FINISHED, reason
        self.stop_reasons[reason] += 1
        self.finished_count += 1
        if seq in self.running_seqs:
            self.running_seqs.remove(seq)
        if seq.slot_id >= 0:
            self.slots[seq.slot_id] = None
            self.free_slots.append(seq.slot_id)
            seq.slot_id = -1
        if seq.output_queue is not None:
            seq.output_queue.put(None)

    # ------------------------------------------------------------------ scheduling
    def _schedule(self) -> Tuple[List[SequenceState], List[Tuple[SequenceState, List[int]]]]:
        decode = list(self.running_seqs)
        budget = self.max_batch_tokens - len(decode)
        while self.waiting_queue and self.free_slots:
            seq = self.waiting_queue.popleft()
            slot = self.free_slots.popleft()
            seq.slot_id, self.slots[slot] = slot, seq
            seq.status = SeqStatus.PREFILLING
            self._init_slot_state(seq, slot)
            self.prefilling_seqs.append(seq)
        prefill: List[Tuple[SequenceState, List[int]]] = []
        for seq in self.prefilling_seqs:
            if seq.pending_logits is not None:
                prefill.append((seq, []))
                continue
            if budget <= 0:
                break
            remaining = len(seq.prompt_tokens) - seq.prefill_offset
            take = min(remaining, self.prefill_chunk_size, budget)
            prefill.append((seq, seq.prompt_tokens[seq.prefill_offset:seq.prefill_offset + take]))
            budget -= take
        return decode, prefill

    def _emit(self, seq: SequenceState, logits_row: torch.Tensor) -> Tuple[Union[int, str], int]:
        proc = None
        if seq.enforcer is not None and not seq.enforcer_finished:
            proc = seq.enforcer.mask_logits
        tok, _ = self.sampler.sample(logits_row, seq.temperature, seq.top_p, seq.top_k, seq.logit_bias, proc)
        seq.generated_tokens.append(tok)
        seq.last_token_id = tok
        if seq.enforcer is not None and not seq.enforcer_finished:
            seq.enforcer.update(tok)
            seq.enforcer_finished = bool(seq.enforcer.is_finished())
        if seq.output_queue is not None:
            seq.output_queue.put(tok)
        eos = seq.eos_token_id if seq.eos_token_id is not None else getattr(self.tokenizer, "eos_token_id", None)
        if eos is not None and tok == eos:
            self._finish_sequence(seq, "eos")
        elif seq.enforcer is not None and seq.enforcer_finished:
            self._finish_sequence(seq, "schema_complete")
        elif seq.num_generated >= seq.max_new_tokens:
            self._finish_sequence(seq, "length")
        elif seq.stop and self.tokenizer is not None:
            seq.generated_text = self.tokenizer.decode(seq.generated_tokens)
            if any(s in seq.generated_text for s in seq.stop):
                self._finish_sequence(seq, "stop")
        if os.environ.get("RWKV_DEBUG_DECODE") == "1":
            print(f"[decode] seq {seq.seq_id} token {tok} status {seq.status.value}")
        return seq.seq_id, tok

    def _execute_decode(self, batch: List[SequenceState]) -> List[Tuple[Union[int, str], int]]:
        if not batch:
            return []
        ids = torch.tensor([[s.last_token_id] for s in batch], dtype=torch.long, device=self.device)
        logits = self._model_forward_with_state(ids, [s.slot_id for s in batch])
        return [self._emit(s, logits[i]) for i, s in enumerate(batch)]

    def _execute_prefill(self, batch: List[Tuple[SequenceState, List[int]]]) -> List[Tuple[Union[int, str], int]]:
        out: List[Tuple[Union[int, str], int]] = []
        groups: Dict[int, List[Tuple[SequenceState, List[int]]]] = collections.defaultdict(list)
        for seq, chunk in batch:
            groups[len(chunk)].append((seq, chunk))
        for n_tok, members in groups.items():
            if n_tok == 0:     # full cache hit: sample straight from the cached logits
                for seq, _ in members:
                    logits_row, seq.pending_logits = seq.pending_logits, None
                    self._promote(seq)
                    out.append(self._emit(seq, logits_row))
                continue
            ids = torch.tensor([c for _, c in members], dtype=torch.long, device=self.device)
            logits = self._model_forward_with_state(ids, [s.slot_id for s, _ in members])
            for i, (seq, chunk) in enumerate(members):
                seq.prefill_offset += len(chunk)
                if seq.prefill_offset >= len(seq.prompt_tokens):
                    if self.state_cache is not None and self.state_cache.is_enabled():
                        self.state_cache.create_checkpoints(seq.prompt_tokens, None,
                                                            self._back_state_from_slot(seq.slot_id), logits[i])
                    self._promote(seq)
                    out.append(self._emit(seq, logits[i]))
        return out

    def _promote(self, seq: SequenceState) -> None:
        if seq in self.prefilling_seqs:
            self.prefilling_seqs.remove(seq)
        seq.status = SeqStatus.RUNNING
        self.running_seqs.append(seq)

    # ------------------------------------------------------------------ stepping
    def step_sync(self) -> List[Tuple[Union[int, str], int]]:
        """One scheduling round: decode every running sequence, then advance prefills.  Retries (up to
        10 times, after emptying the allocator cache) when CUDA reports out of memory."""
        for attempt in range(10):
            try:
                decode, prefill = self._schedule()
                return self._execute_decode(decode) + self._execute_prefill(prefill)
            except torch.cuda.OutOfMemoryError:
                if attempt == 9:
                    raise
                torch.cuda.empty_cache()
                time.sleep(0.05 * (attempt + 1))
        return []

    async def step_async(self):
        return self.step_sync()

    def run_to_completion_sync(self, max_steps: int = 100000, stall_steps: int = 500, stall_seconds: float = 60.0
                               ) -> Iterator[List[Tuple[Union[int, str], int]]]:
        steps, idle, t_progress = 0, 0, time.time()
        while self.has_pending_work():
            produced = self.step_sync()
            steps += 1
            if produced:
                idle, t_progress = 0, time.time()
            else:
                idle += 1
            yield produced
            if steps >= max_steps:
                raise RuntimeError(f"scheduler exceeded {max_steps} steps: {self.get_stats()}")
            if idle >= stall_steps and time.time() - t_progress > stall_seconds:
                raise RuntimeError(f"scheduler made no progress for {idle} steps: {self.get_stats()}")


def create_scheduler_core(model, tokenizer, max_batch_size: int = 64, max_batch_tokens: int = 8192,
                          prefill_chunk_size: int = 512, state_cache=None, use_state_cache: bool = False,
                          max_cache_memory_gb: float = 4.0) -> SchedulerCore:
    """``state_cache``: a ready :class:`StateCache` (the reference's argument); ``use_state_cache=True`` builds one."""
    cache = state_cache
    if cache is None and use_state_cache:
        from .state_cache import create_state_cache

        cache = create_state_cache(model, max_cache_memory_gb)
    return SchedulerCore(model, tokenizer, max_batch_size, max_batch_tokens, prefill_chunk_size, cache)
