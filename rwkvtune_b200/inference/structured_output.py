"""JSON-constrained decoding on top of ``lm-format-enforcer``
(``rwkvtune/inference/structured_output.py:39-441``).

``JsonSchemaEnforcer`` / ``JsonObjectEnforcer`` expose ``mask_logits`` (set disallowed ids to -inf),
``update(token_id)`` and ``is_finished()``; ``create_enforcer(response_format)`` maps OpenAI-style
``{"type": "json_schema" | "json_object" | "text"}`` onto them.  The allowed-id set of a parser state
is turned into a device mask once and cached, so repeated states cost one ``torch.where``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

import torch

try:
    from lmformatenforcer import JsonSchemaParser, TokenEnforcer
    from lmformatenforcer.tokenenforcer import TokenEnforcerTokenizerData

    LM_FORMAT_ENFORCER_AVAILABLE = True
except Exception:   # optional dependency
    LM_FORMAT_ENFORCER_AVAILABLE = False


def build_token_enforcer_tokenizer_data(tokenizer) -> "TokenEnforcerTokenizerData":
    """Vocabulary table for the enforcer, built straight from the byte tokenizer (no dependency on the
    ``transformers`` integration module).  A byte-level vocabulary has no word-start marker, so every
    token is reported as a plain continuation; ids that do not decode to text are left out."""
    special = set(tokenizer.all_special_ids)
    idx2 = getattr(tokenizer, "idx2token", None)
    ids = sorted(idx2.keys()) if idx2 else range(len(tokenizer))
    regular = []
    for tid in ids:
        if tid in special:
            continue
        text = tokenizer.decode([tid])
        if not text or "\ufffd" in text:
            continue
        regular.append((tid, text, False))

    def decode_fn(tokens):
        return tokenizer.decode(list(tokens)).rstrip("\ufffd")

    return TokenEnforcerTokenizerData(regular, decode_fn, tokenizer.eos_token_id, False, len(tokenizer))


def is_structured_output_available() -> bool:
    return LM_FORMAT_ENFORCER_AVAILABLE


class TokenizerAdapter:
    """Adds what lm-format-enforcer expects from a tokenizer: ``all_special_ids``, ``vocab_size``,
    ``convert_ids_to_tokens``, ``get_vocab``.  Low ids that decode to nothing, to U+FFFD or to control
    characters are listed as special so the enforcer never proposes them."""

    def __init__(self, tokenizer):
        self._tokenizer = tokenizer
        self._vocab_size = int(getattr(tokenizer, "vocab_size", 65536))
        special = {getattr(tokenizer, a, None) for a in ("eos_token_id", "bos_token_id", "pad_token_id", "unk_token_id")}
        special.discard(None)
        for tid in range(min(512, self._vocab_size)):
            try:
                s = tokenizer.decode([tid])
            except Exception:
                s = ""
            if not s or s == "�" or (len(s) == 1 and ord(s) < 32 and s not in "\n\r\t"):
                special.add(tid)
        self.all_special_ids = sorted(special)

    def __getattr__(self, name):
        return getattr(self._tokenizer, name)

    def convert_ids_to_tokens(self, ids):
        if isinstance(ids, int):
            return self._tokenizer.decode([ids])
        return [self._tokenizer.decode([i]) for i in ids]

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def __len__(self) -> int:
        return self._vocab_size

    def get_vocab(self) -> Dict[str, int]:
        idx2 = getattr(self._tokenizer, "idx2token", None)
        if idx2:
            return {v.decode("utf-8", errors="replace"): k for k, v in idx2.items()}
        return {self._tokenizer.decode([i]): i for i in range(min(self._vocab_size, 1000))}


class _EnforcerBase:
    def __init__(self, tokenizer, parser):
        if not LM_FORMAT_ENFORCER_AVAILABLE:
            raise ImportError("lm-format-enforcer is required for structured output (pip install lm-format-enforcer)")
        self.tokenizer = tokenizer
        self.adapted_tokenizer = TokenizerAdapter(tokenizer)
        self.tokenizer_data = build_token_enforcer_tokenizer_data(self.adapted_tokenizer)
        self.parser = parser
        self.enforcer = TokenEnforcer(self.tokenizer_data, parser)
        self._generated_tokens: List[int] = []
        self._is_finished = False
        self._invalid: Optional[set] = None
        self._mask_cache: Dict[tuple, torch.Tensor] = {}

    def _get_invalid_tokens(self) -> set:
        if self._invalid is None:
            bad = set()
            idx2 = getattr(self.tokenizer, "idx2token", None)
            ids = idx2.keys() if idx2 else range(self.adapted_tokenizer.vocab_size)
            for tid in ids:
                try:
                    if self.tokenizer.decode([tid]) == "�":
                        bad.add(tid)
                except Exception:
                    bad.add(tid)
            self._invalid = bad
        return self._invalid

    def get_allowed_tokens(self) -> List[int]:
        allowed = self.enforcer.get_allowed_tokens(self._generated_tokens).allowed_tokens or []
        bad = self._get_invalid_tokens()
        return [t for t in allowed if t not in bad]

    def mask_logits(self, logits: torch.Tensor) -> torch.Tensor:
        if self._is_finished:
            return logits
        allowed = self.get_allowed_tokens()
        if not allowed:
            self._is_finished = True
            return logits
        if logits.dim() not in (1, 2):
            raise ValueError(f"unsupported logits shape {tuple(logits.shape)}")
        key = (tuple(allowed), logits.shape[-1], str(logits.device))
        keep = self._mask_cache.get(key)
        if keep is None:
            keep = torch.zeros(logits.shape[-1], dtype=torch.bool, device=logits.device)
            keep[torch.tensor([t for t in allowed if t < logits.shape[-1]], dtype=torch.long, device=logits.device)] = True
            if len(self._mask_cache) < 256:
                self._mask_cache[key] = keep
        return torch.where(keep, logits, torch.full_like(logits, float("-inf")))

    def update(self, token_id: int) -> bool:
        self._generated_tokens.append(int(token_id))
        try:
            if not self.get_allowed_tokens():
                self._is_finished = True
            eos = getattr(self.tokenizer, "eos_token_id", None)
            if eos is not None and token_id == eos:
                self._is_finished = True
        except Exception as exc:
            print(f"[structured output] enforcer update failed, ending the constraint: {exc}")
            self._is_finished = True
        return self._is_finished

    def is_finished(self) -> bool:
        return self._is_finished

    def reset(self) -> None:
        self._generated_tokens = []
        self._is_finished = False


class JsonSchemaEnforcer(_EnforcerBase):
    def __init__(self, tokenizer, schema: Dict[str, Any]):
        if not LM_FORMAT_ENFORCER_AVAILABLE:
            raise ImportError("lm-format-enforcer is required for structured output (pip install lm-format-enforcer)")
        self.schema = schema
        super().__init__(tokenizer, JsonSchemaParser(schema))


class JsonObjectEnforcer(_EnforcerBase):
    """Any syntactically valid JSON value (schema ``None``)."""

    def __init__(self, tokenizer):
        if not LM_FORMAT_ENFORCER_AVAILABLE:
            raise ImportError("lm-format-enforcer is required for structured output (pip install lm-format-enforcer)")
        super().__init__(tokenizer, JsonSchemaParser(None))


def create_enforcer(tokenizer, response_format: Optional[Dict[str, Any]] = None
                    ) -> Optional[Union[JsonSchemaEnforcer, JsonObjectEnforcer]]:
    if response_format is None:
        return None
    kind = response_format.get("type", "text")
    if kind == "text":
        return None
    if kind == "json_object":
        return JsonObjectEnforcer(tokenizer)
    if kind == "json_schema":
        spec = response_format.get("json_schema", {})
        schema = spec.get("schema") or spec.get("schema_", {})
        if not schema:
            raise ValueError("json_schema.schema is required when type is 'json_schema'")
        return JsonSchemaEnforcer(tokenizer, schema)
    raise ValueError(f"unsupported response_format type: {kind}")
