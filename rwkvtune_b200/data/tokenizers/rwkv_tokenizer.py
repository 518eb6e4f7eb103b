"""Greedy longest-match byte tokenizer over the RWKV "world" vocabulary.

Vocabulary lines are ``<id> <python literal (str or bytes)> <byte length>``; ids run 1..65529
and id 0 is unused (it serves as padding).  Behavioural parity with
``rwkvtune/data/tokenizers/rwkv_tokenizer.py:5-174``; the trie here is a flat list of
``dict[int, int]`` transition tables (one per node) rather than a tree of Python objects, and
vocabulary literals are parsed with ``ast.literal_eval`` instead of ``eval``.

When the package's native library is present, encoding runs in it (``csrc/tokenizer_trie.cu``: the same greedy
longest match over a hash-table trie: 190 MB/s against 4.8 MB/s for the Python walk on one core, 64 MB/s once the
ids are back in a Python list; ``encode_batch`` spreads a list of texts over threads and can return numpy arrays,
530 MB/s on 8 cores); the Python tables are then built only if something asks for them.
``RWKVTUNE_NATIVE_TOKENIZER=0`` keeps everything in Python.
"""
from __future__ import annotations

import array
import ast
import ctypes
import os
from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np


class _NativeTrie:
    """Handle on a trie inside the native library; ``None`` from :meth:`open` when the library cannot be used."""

    _lib = None
    _tried = False

    @classmethod
    def _library(cls):
        if not cls._tried:
            cls._tried = True
            if os.environ.get("RWKVTUNE_NATIVE_TOKENIZER", "1") != "0":
                path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "csrc",
                                    "librwkvtune_b200.so")
                try:
                    lib = ctypes.CDLL(path)
                    lib.rwkv_trie_create.restype = ctypes.c_void_p
                    lib.rwkv_trie_destroy.argtypes = [ctypes.c_void_p]
                    lib.rwkv_trie_insert.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
                    lib.rwkv_trie_insert_many.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p,
                                                          ctypes.c_void_p, ctypes.c_int]
                    lib.rwkv_trie_encode.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int64, ctypes.c_void_p]
                    lib.rwkv_trie_encode.restype = ctypes.c_int64
                    lib.rwkv_trie_encode_batch.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int,
                                                           ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
                    cls._lib = lib
                except (OSError, AttributeError):      # not built, built without the trie, or its runtime is missing
                    cls._lib = None
        return cls._lib

    @classmethod
    def open(cls, token2idx: Dict[bytes, int]) -> Optional["_NativeTrie"]:
        lib = cls._library()
        if lib is None:
            return None
        self = cls.__new__(cls)
        self.lib, self.handle = lib, ctypes.c_void_p(lib.rwkv_trie_create())
        toks = list(token2idx.items())
        offsets = array.array("q", [0])
        for t, _ in toks:
            offsets.append(offsets[-1] + len(t))
        ids = array.array("i", [i for _, i in toks])
        blob = b"".join(t for t, _ in toks)
        rc = lib.rwkv_trie_insert_many(self.handle, blob, offsets.buffer_info()[0], ids.buffer_info()[0], len(toks))
        if rc != 0:
            self.close()
            return None
        return self

    def insert(self, tok: bytes, idx: int) -> None:
        self.lib.rwkv_trie_insert(self.handle, tok, len(tok), idx)

    def encode(self, src: bytes) -> List[int]:
        n = len(src)
        if n == 0:
            return []
        out = np.empty(n, dtype=np.int32)       # a token covers at least one byte
        count = self.lib.rwkv_trie_encode(self.handle, src, n, out.ctypes.data)
        if count < 0:
            off = -1 - count
            raise ValueError(f"byte {src[off]!r} at offset {off} is not covered by the vocabulary")
        return out[:count].tolist()

    def encode_batch(self, texts: Sequence[bytes], threads: int, arrays: bool = False):
        offsets = np.zeros(len(texts) + 1, dtype=np.int64)
        np.cumsum([len(t) for t in texts], out=offsets[1:])
        total = int(offsets[-1])
        out = np.empty(max(total, 1), dtype=np.int32)
        counts = np.zeros(max(len(texts), 1), dtype=np.int64)
        self.lib.rwkv_trie_encode_batch(self.handle, b"".join(texts), offsets.ctypes.data, len(texts), out.ctypes.data,
                                        counts.ctypes.data, threads)
        result = []
        for i, t in enumerate(texts):
            c = int(counts[i])
            if c < 0:
                off = -1 - c
                raise ValueError(f"text {i}: byte {t[off]!r} at offset {off} is not covered by the vocabulary")
            ids = out[offsets[i]:offsets[i] + c]
            result.append(ids.copy() if arrays else ids.tolist())
        return result

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.rwkv_trie_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_VOCAB_CACHE: Dict[str, tuple] = {}


def _read_vocab(file_name: str) -> Dict[int, bytes]:
    """Parsed vocabulary file, kept per (path, size, mtime): a process usually builds several tokenizers over the same
    file (trainer, generator, pipeline), and parsing 65 k literals takes longer than everything else in the constructor."""
    st = os.stat(file_name)
    key = (st.st_size, st.st_mtime_ns)
    hit = _VOCAB_CACHE.get(file_name)
    if hit is not None and hit[0] == key:
        return hit[1]
    table: Dict[int, bytes] = {}
    with open(file_name, "r", encoding="utf-8") as fh:
        for line in fh:
            sp1 = line.index(" ")
            sp2 = line.rindex(" ")
            idx = int(line[:sp1])
            tok = ast.literal_eval(line[sp1 + 1:sp2])
            tok = tok.encode("utf-8") if isinstance(tok, str) else tok
            if len(tok) != int(line[sp2 + 1:]):
                raise ValueError(f"vocabulary line for id {idx} has inconsistent byte length")
            table[idx] = tok
    _VOCAB_CACHE[file_name] = (key, table)
    return table


class TRIE_TOKENIZER:
    def __init__(self, file_name: str, eos_token: Optional[Union[str, int]] = None):
        self.file_name = file_name
        self.idx2token: Dict[int, bytes] = dict(_read_vocab(file_name))
        self.token2idx: Dict[bytes, int] = {t: i for i, t in self.idx2token.items()}
        self._build_trie()
        self.vocab_size = max(self.idx2token) + 1
        self._init_eos(eos_token)

    # ------------------------------------------------------------------ trie
    def _build_trie(self) -> None:
        self._native = _NativeTrie.open(self.token2idx)
        self._next: Optional[List[Dict[int, int]]] = None
        self._value: Optional[List[int]] = None
        if self._native is None:
            self._build_python_trie()

    def _build_python_trie(self) -> None:
        self._next, self._value = [{}], [-1]
        for tok, idx in self.token2idx.items():
            self._insert_python(tok, idx)
        for tok, idx in getattr(self, "_extra_tokens", {}).items():
            self._insert_python(tok, idx)

    def _insert(self, tok: bytes, idx: int) -> None:
        if self._native is not None:
            self._native.insert(tok, idx)
        if self._next is not None:
            self._insert_python(tok, idx)

    def _insert_python(self, tok: bytes, idx: int) -> None:
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
        for k in ("_next", "_value", "_native"):
            state.pop(k, None)
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._build_trie()
        for tok, idx in getattr(self, "_extra_tokens", {}).items():
            self._insert(tok, idx)

    # ------------------------------------------------------------------ encode / decode
    def encodeBytes(self, src: bytes) -> List[int]:
        if self._native is not None:
            return self._native.encode(src)
        return self._encode_python(src)

    def encode_batch(self, texts: Sequence[str], num_threads: int = 0, return_arrays: bool = False):
        """Ids of every text of a list; with the native library the texts are spread over ``num_threads`` threads
        (0 = one per core, at most 16).  ``return_arrays=True`` gives int32 numpy arrays instead of lists, which
        skips the conversion that otherwise costs more than the encoding itself."""
        raw = [t.encode("utf-8") for t in texts]
        if self._native is not None:
            threads = num_threads if num_threads > 0 else min(16, os.cpu_count() or 1)
            return self._native.encode_batch(raw, threads, return_arrays)
        out = []
        for i, b in enumerate(raw):
            try:
                out.append(self._encode_python(b))
            except ValueError as exc:
                raise ValueError(f"text {i}: {exc}") from None
        return [np.asarray(o, dtype=np.int32) for o in out] if return_arrays else out

    def _encode_python(self, src: bytes) -> List[int]:
        if self._next is None:
            self._build_python_trie()
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
