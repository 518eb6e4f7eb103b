"""ShareGPT helpers shared by the example scripts.

Covers what ``examples/train_sft_single_gpu.py:33-225`` and ``examples/train_grpo_single_gpu.py:56-216``
of the reference do with a ShareGPT ``.jsonl`` / ``.json`` file: load it, turn a conversation into
pre-shifted ``input_ids`` / ``labels`` with everything but the assistant replies masked, and unroll a
conversation into one GRPO prompt per assistant turn.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterable, List, Optional, Tuple

IGNORE_INDEX = -100
THINK_SKIP = "<think>\n\n</think>"      # empty reasoning block: the model answers directly
USER_ROLES = ("human", "user")
ASSISTANT_ROLES = ("gpt", "assistant")


def load_sharegpt(path: str) -> List[Dict[str, Any]]:
    """One JSON object per line (``.jsonl``) or a single JSON list."""
    with open(path, "r", encoding="utf-8") as f:
        text = f.read().strip()
    if not text:
        return []
    if text[0] == "[":
        return json.loads(text)
    return [json.loads(line) for line in text.splitlines() if line.strip()]


def _turns(conversation: Iterable[Dict[str, Any]]):
    for turn in conversation:
        yield str(turn.get("from", "")).lower(), turn.get("value", "")


def encode_sft_sample(conversation, tokenizer, last_reply_only: bool = False,
                      eos_token_id: Optional[int] = None) -> Dict[str, List[int]]:
    """Tokens of ``System: ..\\n\\nUser: ..<eos>Assistant:<think>\\n\\n</think>reply<eos>...`` shifted by one.

    ``labels[i]`` is the token after ``input_ids[i]``; it is ``-100`` unless that token belongs to an
    assistant reply (only the last reply with ``last_reply_only``).  Without an ``eos_token_id`` the turn
    separator is the text ``"\\n\\n"``.
    """
    turns = list(_turns(conversation))
    last_reply = max((i for i, (role, _) in enumerate(turns) if role in ASSISTANT_ROLES), default=None)
    sep = [eos_token_id] if eos_token_id is not None else tokenizer.encode("\n\n")
    tokens: List[int] = []
    learn: List[bool] = []

    def push(ids, flag):
        tokens.extend(ids)
        learn.extend([flag] * len(ids))

    for i, (role, text) in enumerate(turns):
        if role == "system":
            push(tokenizer.encode(f"System: {text}\n\n"), False)
        elif role in USER_ROLES:
            push(tokenizer.encode(f"User: {text}") + sep + tokenizer.encode(f"Assistant:{THINK_SKIP}"), False)
        elif role in ASSISTANT_ROLES:
            push(tokenizer.encode(text) + sep, (not last_reply_only) or i == last_reply)
    if len(tokens) < 2:
        return {"input_ids": [], "labels": []}
    labels = [tok if keep else IGNORE_INDEX for tok, keep in zip(tokens[1:], learn[1:])]
    return {"input_ids": tokens[:-1], "labels": labels}


def build_sft_dataset(records, tokenizer, max_length: int, last_reply_only: bool = False,
                      eos_token_id: Optional[int] = None, min_length: int = 10) -> List[Dict[str, List[int]]]:
    out, skipped = [], 0
    for rec in records:
        conv = rec.get("conversations") or []
        sample = encode_sft_sample(conv, tokenizer, last_reply_only, eos_token_id) if conv else {"input_ids": []}
        if len(sample["input_ids"]) < min_length:
            skipped += 1
            continue
        out.append({k: v[:max_length] for k, v in sample.items()})
    lengths = [len(s["input_ids"]) for s in out] or [0]
    print(f"[data] {len(out)} samples ({skipped} skipped); tokens min/avg/max = "
          f"{min(lengths)}/{sum(lengths) / len(lengths):.0f}/{max(lengths)}")
    return out


def split_conversation(conversation) -> Tuple[str, List[Tuple[str, str]]]:
    """``(system prompt, [(user, assistant), ...])`` in order; a user turn without a reply is dropped."""
    system, pairs, pending = "", [], None
    for role, text in _turns(conversation):
        if role == "system" and not system:
            system = text
        elif role in USER_ROLES:
            pending = text
        elif role in ASSISTANT_ROLES and pending is not None:
            pairs.append((pending, text))
            pending = None
    return system, pairs


ROLEPLAY_INSTRUCTIONS = (
    "**Role:** NPC in an interactive story  \n"
    "**Task:** Respond in character to the user's input  \n"
    "**Tone:** Immersive, concise, consistent with established context  \n"
    "**Length:** ~30 words  \n"
    "**Format:**  \n"
    "- Use *asterisks* for actions  \n"
    "- Reply directly, no greetings or explanations  \n"
    "- No extra formatting or meta-commentary  \n"
    "- Never use quotation marks around speech  \n"
    "- Never use parentheses  \n"
    "- Never start with a role prefix like \"Name:\"  \n"
    "**Example:**  \n"
    "*leans closer with a crooked smile* A better idea than movie night? Now I'm curious... you'd better show me.\n"
    "**Roleplay Background:**\n"
)


def build_grpo_dataset(records, tokenizer, max_prompt_length: int = 1024, min_prompt_tokens: int = 16,
                       instructions: str = ROLEPLAY_INSTRUCTIONS) -> List[Dict[str, Any]]:
    """One sample per assistant turn: the history so far ending in ``Assistant: <think`` as ``prompt`` /
    ``input_ids`` (truncated to ``max_prompt_length``), the recorded reply as ``ground_truth_answer``."""
    samples = []
    for session, rec in enumerate(records):
        system, pairs = split_conversation(rec.get("conversations") or [])
        if not pairs:
            continue
        history = "System: " + instructions + (("\n\n" + system.strip()) if system else "") + "\n\n"
        for turn, (user, reply) in enumerate(pairs):
            prompt = f"{history}User: {user}\n\nAssistant: <think"
            ids = tokenizer.encode(prompt)[:max_prompt_length]
            if len(ids) >= min_prompt_tokens:
                samples.append({"prompt": prompt, "input_ids": ids, "ground_truth_answer": reply,
                                "session_index": session, "turn_index": turn})
            history += f"User: {user}\n\nAssistant: {reply}\n\n"
    if not samples:
        raise RuntimeError("no GRPO samples could be built from the data file")
    lengths = [len(s["input_ids"]) for s in samples]
    print(f"[data] {len(samples)} GRPO prompts; tokens min/avg/max = "
          f"{min(lengths)}/{sum(lengths) / len(lengths):.0f}/{max(lengths)}")
    return samples


def first_user_prompt(conversation) -> str:
    """Prompt for a generation smoke test: system + first user turn, ready for the assistant to continue."""
    system, pairs = split_conversation(conversation)
    user = pairs[0][0] if pairs else next((t for r, t in _turns(conversation) if r in USER_ROLES), "")
    head = f"System: {system}\n\n" if system else ""
    return f"{head}User: {user}\n\nAssistant:{THINK_SKIP}"


def first_reference(conversation) -> str:
    _, pairs = split_conversation(conversation)
    return pairs[0][1] if pairs else ""
