"""Text-level splitting around special tokens (``<|im_start|>`` and friends).

Special tokens must be matched on the *text* before byte-level tokenisation so that they map
to their reserved ids instead of being spelled out (reference:
``rwkvtune/data/tokenizers/special_token_handler.py:13-216``).  A sorted-by-length scan
replaces the reference's character trie; the longest special token starting at a position wins.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Sequence


class SpecialTokenTrie:
    def __init__(self) -> None:
        self._tokens: List[str] = []
        self._first_chars = set()

    def add(self, word: str) -> None:
        if word and word not in self._tokens:
            self._tokens.append(word)
            self._tokens.sort(key=len, reverse=True)
            self._first_chars.add(word[0])

    def __len__(self) -> int:
        return len(self._tokens)

    def split(self, text: str) -> List[str]:
        """Split ``text`` into pieces such that every special token is its own piece."""
        if not self._tokens or not text:
            return [text] if text else []
        out: List[str] = []
        start = i = 0
        n = len(text)
        while i < n:
            if text[i] in self._first_chars:
                hit = next((tok for tok in self._tokens if text.startswith(tok, i)), None)
                if hit is not None:
                    if i > start:
                        out.append(text[start:i])
                    out.append(hit)
                    i += len(hit)
                    start = i
                    continue
            i += 1
        if start < n:
            out.append(text[start:])
        return out


def encode_with_special_tokens(text: str, base_encode: Callable[[str], List[int]], special_tokens: Dict[str, int],
                               trie: SpecialTokenTrie = None) -> List[int]:
    if trie is None:
        trie = SpecialTokenTrie()
        for tok in special_tokens:
            trie.add(tok)
    ids: List[int] = []
    for piece in trie.split(text):
        if piece in special_tokens:
            ids.append(special_tokens[piece])
        else:
            ids.extend(base_encode(piece))
    return ids


def decode_with_special_tokens(token_ids: Sequence[int], base_decode: Callable[[List[int]], str],
                               id_to_special: Dict[int, str], skip_special_tokens: bool = False) -> str:
    parts: List[str] = []
    run: List[int] = []
    for t in token_ids:
        t = int(t)
        if t in id_to_special:
            if run:
                parts.append(base_decode(run))
                run = []
            if not skip_special_tokens:
                parts.append(id_to_special[t])
        else:
            run.append(t)
    if run:
        parts.append(base_decode(run))
    return "".join(parts)
