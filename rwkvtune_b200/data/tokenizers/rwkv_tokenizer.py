"""Greedy longest-match byte tokenizer over the RWKV "world" vocabulary.

Vocabulary lines are ``<id> <python literal (str or bytes)> <byte length>``; ids run 1..65529
and id 0 is unused (it serves as padding).  Behavioural parity with
``rwkvtune/data/tokenizers/rwkv_tokenizer.py:5-174``; the trie here is a flat list of
``dict[int, int]`` transition tables (one per node) rather than a tree of Python objects, and
vocabulary literals are parsed with ``ast.literal_eval`` instead of ``eval``.
"""
from __future__ import annotations

import ast
import os
from typing import Dict, Iterable, List, Optional, Sequence, Union


class TRIE_TOKENIZER:
    def __init__(self, file_name: str, eos_token: Optional[Union[str, int]] = None):
        self.file_name = file_name
        self.idx2token: Dict[int, bytes] = {}
        with open(file_name, "r", encoding="utf-8") as fh:
            for line in fh:
                sp1 = line.index(" ")
                sp2 = line.rindex(" ")
                idx = int(line[:sp1])
                tok = ast.literal_eval(line[sp1 + 1:sp2])
                tok = tok.encode("utf-8") if isinstance(tok, str) else tok
                if len(tok) != int(line[sp2 + 1:]):
                    raise ValueError(f"vocabulary line for id {idx} has inconsistent byte length")
                self.idx2token[idx] = tok
        self.token2idx: Dict[bytes, int] = {t: i for i, t in self.idx2token.items()}
        self._build_trie()
        self.vocab_size = max(self.idx2token) + 1
        self._init_eos(eos_token)

    # ------------------------------------------------------------------ trie
    def _build_trie(self) -> None:
        self._next: List[Dict[int, int]] = [{}]
        self._value: List[int] = [-1]
        for tok, idx in self.token2idx.items():
            self._insert(tok, idx)

    def _insert(self, tok: bytes, idx: int) -> None:
        node = 0
        nxt, val = self._next, self._value
        for b in tok:
            child = nxt[node].get(b)
            if child is None:
                child = len(nxt)
                nxt[node][b] = child
                nxt.append({})
                val.append(-1)
            node = child
        val[node] = idx

    def _init_eos(self, eos_token: Optional[Union[str, int]]) -> None:
        if eos_token is None:
            eos_token = "\n\n"
        if isinstance(eos_token, int):
            self.eos_token_id = eos_token
            self.eos_token = self.idx2token.get(eos_token, b"").decode("utf-8", errors="replace")
        else:
            self.eos_token = eos_token
            ids = self.encodeBytes(eos_token.encode("utf-8"))
            self.eos_token_id = ids[0] if len(ids) == 1 else (ids[-1] if ids else None)

    # ------------------------------------------------------------------ pickling (vocab is re-read)
    def __getstate__(self):
        state = self.__dict__.copy()
        for k in ("_next", "_value"):
            state.pop(k, None)
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._build_trie()
        for tok, idx in getattr(self, "_extra_tokens", {}).items():
            self._insert(tok, idx)

    # ------------------------------------------------------------------ encode / decode
    def encodeBytes(self, src: bytes) -> List[int]:
        out: List[int] = []
        nxt, val = self._next, self._value
        i, n = 0, len(src)
        while i < n:
            node, j, best, best_end = 0, i, -1, i
            while j < n:
                node = nxt[node].get(src[j])
                if node is None:
                    break
                j += 1
                if val[node] >= 0:
                    best, best_end = val[node], j
            if best < 0:
                raise ValueError(f"byte {src[i]!r} at offset {i} is not covered by the vocabulary")
            out.append(best)
            i = best_end
        return out

    def decodeBytes(self, tokens: Iterable[int]) -> bytes:
        return b"".join(self.idx2token[int(t)] for t in tokens)

    def encode(self, src: str) -> List[int]:
        return self.encodeBytes(src.encode("utf-8"))

    def decode(self, tokens: Sequence[int], skip_special_tokens: bool = False) -> str:
        """Tolerant decode: unknown ids are dropped and invalid UTF-8 becomes U+FFFD
        (``rwkv_tokenizer.py:128-164``)."""
        if hasattr(tokens, "tolist"):
            tokens = tokens.tolist()
        debug = os.environ.get("RWKV_DEBUG_DECODE") == "1"
        parts = []
        for t in tokens:
            tok = self.idx2token.get(int(t))
            if tok is None:
                if debug:
                    print(f"[decode] unknown token id {t} skipped")
                continue
            parts.append(tok)
        return b"".join(parts).decode("utf-8", errors="replace")

    def get_vocab_size(self) -> int:
        return self.vocab_size

    def printTokens(self, tokens: Iterable[int]) -> None:
        for t in tokens:
            tok = self.idx2token[int(t)]
            try:
                shown = tok.decode("utf-8")
            except UnicodeDecodeError:
                shown = tok
            print(f"{shown!r}{t} ", end="")
        print()
