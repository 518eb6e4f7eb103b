"""Text-level splitting around special tokens (``<|im_start|>`` and friends).

Special tokens must be matched on the *text* before byte-level tokenisation so that they map
to their reserved ids instead of being spelled out (reference:
``rwkvtune/data/tokenizers/special_token_handler.py:13-216``).  A sorted-by-length scan
replaces the reference's character trie; the longest special token starting at a position wins.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union


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


def _codec(tokenizer, name: str) -> Callable:
    """``tokenizer.encode`` / ``tokenizer.decode``, or ``tokenizer`` itself when a bare function is passed."""
    return getattr(tokenizer, name) if hasattr(tokenizer, name) else tokenizer


def encode_with_special_tokens(text: str, tokenizer, additional_special_tokens: Dict[str, Union[int, List[int]]],
                               trie: Optional[SpecialTokenTrie] = None) -> List[int]:
    """Encode ``text`` with every special token mapped to its reserved id - or id sequence, when the mapping's value
    is a list - and everything between them encoded by ``tokenizer`` (an object with ``encode`` or the function
    itself).  Call convention of ``special_token_handler.py:118-159``; ``trie`` lets a caller reuse a prepared
    splitter."""
    encode = _codec(tokenizer, "encode")
    if not additional_special_tokens:
        return list(encode(text))
    if trie is None:
        trie = SpecialTokenTrie()
        for tok in additional_special_tokens:
            trie.add(tok)
    ids: List[int] = []
    for piece in trie.split(text):
        hit = additional_special_tokens.get(piece)
        if hit is None:
            ids.extend(encode(piece))
        elif isinstance(hit, (list, tuple)):
            ids.extend(int(t) for t in hit)
        else:
            ids.append(int(hit))
    return ids


def decode_with_special_tokens(token_ids: Sequence[int], tokenizer, additional_special_tokens: Dict[str, Union[int, List[int]]],
                               reverse_mapping: Optional[Dict[Tuple[int, ...], str]] = None,
                               skip_special_tokens: bool = False) -> str:
    """Inverse of :func:`encode_with_special_tokens` (``special_token_handler.py:162-216``): id sequences of special
    tokens (longest first, up to 10 ids) turn back into their strings, everything else goes through ``tokenizer``.
    Unlike the reference, which decodes unmatched ids one at a time, the ids between two special tokens are decoded
    as one run, so a character whose bytes span several tokens survives."""
    decode = _codec(tokenizer, "decode")
    ids = [int(t) for t in token_ids]
    if not additional_special_tokens:
        return decode(ids)
    if reverse_mapping is None:
        reverse_mapping = {(tuple(int(t) for t in v) if isinstance(v, (list, tuple)) else (int(v),)): k
                           for k, v in additional_special_tokens.items()}
    longest = min(10, max((len(k) for k in reverse_mapping), default=1))
    parts: List[str] = []
    run: List[int] = []
    i = 0
    while i < len(ids):
        hit = next((n for n in range(min(longest, len(ids) - i), 0, -1) if tuple(ids[i:i + n]) in reverse_mapping), 0)
        if hit:
            if run:
                parts.append(decode(run))
                run = []
            if not skip_special_tokens:
                parts.append(reverse_mapping[tuple(ids[i:i + hit])])
            i += hit
        else:
            run.append(ids[i])
            i += 1
    if run:
        parts.append(decode(run))
    return "".join(parts)
