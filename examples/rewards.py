"""Reward functions of the role-play GRPO example.

Seven rule-based rewards, each mapping ``(prompts, completions, **dataset_fields)`` to one score in
``[-1, 1]`` per completion, with the default weights of the reference example
(``examples/train_grpo_single_gpu.py:249-411``).  The prompt ends in ``<think`` so a well-formed
completion is ``reasoning</think>reply\\n\\n``.
"""
from __future__ import annotations

import re
from typing import Callable, List, Sequence, Tuple

THINK_CLOSE = "</think>"
_QUOTES = set('"“”')
_PARENS = set("()（）")
_ROLE_PREFIX = re.compile(r"^\s*\w[\w\s]{0,20}:")


def band_score(x: int, soft_min: int, lo: int, hi: int, soft_max: int) -> float:
    """1 inside ``[lo, hi]``, linear ramps down to 0 at the soft limits, -0.5 outside them (and for x <= 0)."""
    if x <= 0 or x < soft_min or x > soft_max:
        return -0.5
    if lo <= x <= hi:
        return 1.0
    if x < lo:
        return (x - soft_min) / max(1.0, lo - soft_min)
    return (soft_max - x) / max(1.0, soft_max - hi)


def split_think(completion: str) -> Tuple[str, str]:
    text = (completion or "").strip()
    cut = text.find(THINK_CLOSE)
    if cut < 0:
        return "", text
    return text[:cut].strip(), text[cut + len(THINK_CLOSE):].strip()


def _words(text: str) -> set:
    return {w for w in re.findall(r"\w+", text.lower()) if len(w) > 2}


def build_reward_functions(tokenizer) -> Tuple[List[Callable], List[float]]:
    n_tokens = lambda text: len(tokenizer.encode(text)) if text else 0
    structured = lambda c: bool(c) and THINK_CLOSE in c

    def per_completion(fn, missing):
        def reward(prompts: Sequence[str], completions: Sequence[str], **fields) -> List[float]:
            return [missing if c is None else fn(c, i, fields) for i, c in enumerate(completions)]
        return reward

    def has_think(c, i, fields):
        return 1.0 if structured(c) else -1.0

    def think_len(c, i, fields):
        return band_score(n_tokens(split_think(c)[0]), 300, 500, 1000, 1200) if structured(c) else -0.5

    def reply_len(c, i, fields):
        if not structured(c):
            return -0.5
        n = n_tokens(split_think(c)[1])
        if n > 100:
            return -1.0
        if n > 50:
            return -0.5
        return band_score(n, 5, 10, 30, 50)

    def actions_style(c, i, fields):
        reply = split_think(c)[1]
        stars = reply.count("*")
        if stars < 2:
            return -0.5 if stars == 1 else -0.3
        if stars % 2:
            return -0.5
        parts = reply.split("*")
        action = any(p.strip() for p in parts[1::2])
        speech = any(p.strip() for p in parts[0::2])
        return 1.0 if (action and speech) else (0.3 if (action or speech) else -0.3)

    def similarity(c, i, fields):
        truth = (fields.get("ground_truth_answer") or [None] * (i + 1))[i]
        if not isinstance(truth, str) or not truth.strip():
            return 0.0
        want, got = _words(truth), _words(split_think(c)[1])
        if not want or not got:
            return -0.3
        return min(1.0, 2.0 * len(want & got) / len(want)) - 0.2

    def format_clean(c, i, fields):
        reply = split_think(c)[1]
        if not reply:
            return 0.0
        faults = (any(ch in _QUOTES for ch in reply) + any(ch in _PARENS for ch in reply)
                  + bool(_ROLE_PREFIX.search(reply)))
        return (1.0, -0.5, -1.0, -1.0)[faults]

    def eos_ending(c, i, fields):
        return 1.0 if c.rstrip(" ").endswith("\n\n") else -0.5

    table = [(has_think, -1.0, 1.0), (think_len, -0.5, 0.5), (reply_len, -0.5, 0.6), (actions_style, -0.5, 0.8),
             (similarity, -0.5, 0.5), (format_clean, 0.0, 0.8), (eos_ending, -1.0, 1.2)]
    fns = []
    for fn, missing, _ in table:
        wrapped = per_completion(fn, missing)
        wrapped.__name__ = f"reward_{fn.__name__}"
        fns.append(wrapped)
    return fns, [w for _, _, w in table]
