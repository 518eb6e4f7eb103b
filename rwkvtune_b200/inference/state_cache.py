"""Prefix cache of recurrent states.

An RWKV state summarises an arbitrarily long prefix in O(1) memory, so caching the state after a
shared system prompt (or a whole prompt) lets later requests skip that part of the prefill.  API
parity with ``rwkvtune/inference/state_cache.py:26-734``: ``CacheLevel`` (none / exact / prefix),
``CacheConfig``, ``AutoConfig`` sizing, ``StateCache.lookup(tokens) -> (cached_len, state, logits)``,
``create_checkpoints``, LRU eviction by bytes and entry count, CPU storage, statistics.

Index: a token trie stored as one ``dict[(node, token)] -> node`` map; entries hang off trie nodes.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch


class CacheLevel(Enum):
    NONE = "none"
    EXACT = "exact"
    PREFIX = "prefix"


class EvictionPolicy(Enum):
    LRU = "lru"


@dataclass
class CacheConfig:
    max_cache_memory_gb: float = 4.0
    max_cache_entries: Optional[int] = None
    cache_level: CacheLevel = CacheLevel.PREFIX
    eviction_policy: EvictionPolicy = EvictionPolicy.LRU
    cache_first_message: bool = True

    def __post_init__(self) -> None:
        if self.max_cache_memory_gb <= 0:
            raise ValueError("max_cache_memory_gb must be positive")


@dataclass(eq=False)
class CachedState:
    tokens: Tuple[int, ...]
    state: List[Dict[str, torch.Tensor]]
    output: torch.Tensor
    memory_bytes: int
    checkpoint_type: str = "full_prompt"
    created_at: float = field(default_factory=time.time)
    last_access: float = field(default_factory=time.time)
    access_count: int = 0

    def update_access(self) -> None:
        self.last_access = time.time()
        self.access_count += 1


class CacheIndex:
    def __init__(self) -> None:
        self._edges: Dict[Tuple[int, int], int] = {}
        self._entry: Dict[int, CachedState] = {}
        self._parent: Dict[int, Tuple[int, int]] = {}
        self._children: Dict[int, int] = {}
        self._next_node = 1
        self._bytes = 0

    def insert(self, tokens: Sequence[int], cached: CachedState) -> None:
        node = 0
        for t in tokens:
            nxt = self._edges.get((node, t))
            if nxt is None:
                nxt = self._next_node
                self._next_node += 1
                self._edges[(node, t)] = nxt
                self._parent[nxt] = (node, t)
                self._children[node] = self._children.get(node, 0) + 1
            node = nxt
        old = self._entry.get(node)
        if old is not None:
            self._bytes -= old.memory_bytes
        self._entry[node] = cached
        self._bytes += cached.memory_bytes

    def _walk(self, tokens: Sequence[int]):
        node = 0
        for i, t in enumerate(tokens):
            node = self._edges.get((node, t))
            if node is None:
                return
            yield i + 1, node

    def find_exact(self, tokens: Sequence[int]) -> Optional[CachedState]:
        last = None
        for depth, node in self._walk(tokens):
            last = (depth, node)
        if last is not None and last[0] == len(tokens):
            return self._entry.get(last[1])
        return None

    def find_longest_cached_prefix(self, tokens: Sequence[int]) -> Tuple[int, Optional[CachedState]]:
        best: Tuple[int, Optional[CachedState]] = (0, None)
        for depth, node in self._walk(tokens):
            hit = self._entry.get(node)
            if hit is not None:
                best = (depth, hit)
        return best

    def remove(self, cached: CachedState) -> bool:
        last = None
        for depth, node in self._walk(cached.tokens):
            last = (depth, node)
        if last is None or last[0] != len(cached.tokens) or self._entry.get(last[1]) is not cached:
            return False
        node = last[1]
        del self._entry[node]
        self._bytes -= cached.memory_bytes
        while node != 0 and node not in self._entry and self._children.get(node, 0) == 0:
            parent, tok = self._parent.pop(node)
            del self._edges[(parent, tok)]
            self._children[parent] -= 1
            node = parent
        return True

    def total_memory_bytes(self) -> int:
        return self._bytes

    def __len__(self) -> int:
        return len(self._entry)

    def get_all_entries(self) -> List[CachedState]:
        return list(self._entry.values())


class AutoConfig:
    @staticmethod
    def estimate_state_size(model, device: str = "cpu") -> int:
        cfg = model.config
        H, N = cfg.dim_att // cfg.head_size_a, cfg.head_size_a
        per_layer = 2 * cfg.n_embd * 4 + H * N * N * 4
        return cfg.n_layer * per_layer + cfg.vocab_size * 4

    @staticmethod
    def calculate(max_memory_gb: float, model_state_size_bytes: int, safety_factor: float = 0.9) -> CacheConfig:
        """Entry count that fits ``safety_factor`` of the budget (``rwkvtune/inference/state_cache.py:231-259``)."""
        budget = int(max_memory_gb * 1e9 * safety_factor)
        entries = max(1, budget // max(int(model_state_size_bytes), 1))
        return CacheConfig(max_cache_memory_gb=max_memory_gb, max_cache_entries=entries)


@dataclass
class CacheStats:
    total_hits: int = 0
    total_misses: int = 0
    exact_hits: int = 0
    prefix_hits: int = 0
    evictions: int = 0
    inserts: int = 0
    tokens_saved: int = 0
    entries_by_type: Dict[str, int] = field(default_factory=dict)

    @property
    def hit_rate(self) -> float:
        n = self.total_hits + self.total_misses
        return self.total_hits / n if n else 0.0

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.__dict__)
        d["hit_rate"] = self.hit_rate
        return d


class StateCache:
    def __init__(self, model, config: Optional[CacheConfig] = None, auto_config: bool = True,
                 max_cache_memory_gb: float = 4.0, verbose: bool = False):
        self.model = model
        self.device = next(model.parameters()).device
        if config is not None:
            self.config = config
        elif auto_config:
            self.config = AutoConfig.calculate(max_cache_memory_gb, AutoConfig.estimate_state_size(model))
        else:
            self.config = CacheConfig(max_cache_memory_gb=max_cache_memory_gb)
        self.index = CacheIndex()
        self.stats = CacheStats()
        self._lock = threading.RLock()
        if verbose:
            print(f"[state cache] level={self.config.cache_level.value} limit={self.config.max_cache_memory_gb:.1f} GB "
                  f"entries<={self.config.max_cache_entries}")

    # ------------------------------------------------------------------ lookup / insert
    def lookup(self, tokens: Sequence[int]):
        if self.config.cache_level == CacheLevel.NONE:
            self.stats.total_misses += 1
            return 0, None, None
        with self._lock:
            if self.config.cache_level == CacheLevel.EXACT:
                hit = self.index.find_exact(tokens)
                pos = len(tokens) if hit is not None else 0
            else:
                pos, hit = self.index.find_longest_cached_prefix(tokens)
            if hit is None:
                self.stats.total_misses += 1
                return 0, None, None
            hit.update_access()
            self.stats.total_hits += 1
            self.stats.tokens_saved += pos
            if pos == len(tokens):
                self.stats.exact_hits += 1
            else:
                self.stats.prefix_hits += 1
            return pos, self._to_device(hit.state), hit.output.to(self.device)

    def put(self, tokens: Sequence[int], state: List[Dict[str, torch.Tensor]], output: torch.Tensor,
            checkpoint_type: str = "full_prompt") -> None:
        with self._lock:
            cpu_state = [{k: v.detach().to("cpu", copy=True) for k, v in layer.items()} for layer in state]
            out = output.detach().to("cpu", copy=True)
            nbytes = sum(v.numel() * v.element_size() for layer in cpu_state for v in layer.values())
            nbytes += out.numel() * out.element_size()
            self.index.insert(tuple(tokens), CachedState(tuple(tokens), cpu_state, out, nbytes, checkpoint_type))
            self.stats.inserts += 1
            self.stats.entries_by_type[checkpoint_type] = self.stats.entries_by_type.get(checkpoint_type, 0) + 1
            self._maybe_evict()

    @torch.no_grad()
    def create_checkpoints(self, tokens: Sequence[int], messages=None,
                           state: Optional[List[Dict[str, torch.Tensor]]] = None, output: Optional[torch.Tensor] = None,
                           chunk_size: int = 2048, system_prompt_len: Optional[int] = None) -> int:
        """Cache the state after the first message and after the full prompt.  The first-message boundary is
        ``system_prompt_len`` tokens when given (an int passed as ``messages`` means the same); with a message list
        it is estimated from the share of characters in the first message, as the reference does
        (``rwkvtune/inference/state_cache.py:458-589``).  If ``state`` / ``output`` for the full prompt are supplied
        they are stored as they are; the prefix state is computed by running the model."""
        if self.config.cache_level == CacheLevel.NONE:
            return 0
        made = 0
        tokens = list(tokens)
        if isinstance(messages, int):
            system_prompt_len, messages = messages, None
        if system_prompt_len is None and messages:
            chars = [len(m.get("content", "")) for m in messages]
            if sum(chars) > 0 and len(tokens) > 1:
                system_prompt_len = max(1, min(int(len(tokens) * chars[0] / sum(chars)), len(tokens) - 1))
        cuts = []
        if self.config.cache_first_message and system_prompt_len and 0 < system_prompt_len < len(tokens):
            cuts.append((system_prompt_len, "system_prompt"))
        cuts.append((len(tokens), "full_prompt"))
        for cut, kind in cuts:
            if self.index.find_exact(tokens[:cut]) is not None:
                continue
            if cut == len(tokens) and state is not None and output is not None:
                st, out = state, output
            else:
                st, out = self._run(tokens[:cut], chunk_size)
            self.put(tokens[:cut], st, out, kind)
            made += 1
        return made

    def _run(self, tokens: List[int], chunk_size: int):
        st = None
        logits = None
        for c0 in range(0, len(tokens), chunk_size):
            ids = torch.tensor([tokens[c0:c0 + chunk_size]], dtype=torch.long, device=self.device)
            logits, st = self.model.forward_with_state(ids, st, last_only=True)
        return st, logits[0, -1].float()

    # ------------------------------------------------------------------ eviction / misc
    def _maybe_evict(self) -> None:
        limit = int(self.config.max_cache_memory_gb * (1 << 30))
        cap = self.config.max_cache_entries
        while len(self.index) > 1 and (self.index.total_memory_bytes() > limit or (cap and len(self.index) > cap)):
            if not self._evict_one():
                break

    def _evict_one(self) -> bool:
        entries = self.index.get_all_entries()
        if not entries:
            return False
        victim = min(entries, key=lambda e: e.last_access)
        ok = self.index.remove(victim)
        if ok:
            self.stats.evictions += 1
            t = victim.checkpoint_type
            self.stats.entries_by_type[t] = max(0, self.stats.entries_by_type.get(t, 1) - 1)
        return ok

    def _to_device(self, state):
        return [{k: v.to(self.device, copy=True) for k, v in layer.items()} for layer in state]

    def get_stats(self) -> Dict[str, Any]:
        d = self.stats.to_dict()
        d.update(entries=len(self.index), memory_bytes=self.index.total_memory_bytes())
        return d

    def clear(self) -> None:
        with self._lock:
            self.index = CacheIndex()

    def is_enabled(self) -> bool:
        return self.config.cache_level != CacheLevel.NONE


def create_state_cache(model, max_cache_memory_gb: float = 4.0, cache_level: str = "prefix",
                       cache_first_message: bool = True, max_cache_entries: Optional[int] = None) -> StateCache:
    cfg = AutoConfig.calculate(max_cache_memory_gb, AutoConfig.estimate_state_size(model))
    cfg.cache_level = CacheLevel(cache_level)
    cfg.cache_first_message = cache_first_message
    if max_cache_entries is not None:
        cfg.max_cache_entries = max_cache_entries
    return StateCache(model, config=cfg)
