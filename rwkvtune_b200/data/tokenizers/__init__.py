"""Tokenizers for RWKV models (``rwkvtune/data/tokenizers/__init__.py:1-76``)."""
import os
from typing import Optional

from .auto_tokenizer import AutoTokenizer, RWKVTokenizer, TokenizerConfig
from .rwkv_tokenizer import TRIE_TOKENIZER

__all__ = ["TRIE_TOKENIZER", "AutoTokenizer", "RWKVTokenizer", "TokenizerConfig", "get_tokenizer", "get_vocab_path"]


def get_vocab_path(vocab_name: str = "rwkv_vocab_v20230424.txt") -> str:
    path = os.path.join(os.path.dirname(__file__), "vocab", vocab_name)
    if not os.path.exists(path):
        raise FileNotFoundError(f"vocabulary file not found: {path}")
    return path


def get_tokenizer(vocab_path: Optional[str] = None, vocab_name: str = "rwkv_vocab_v20230424.txt",
                  eos_token=None) -> TRIE_TOKENIZER:
    return TRIE_TOKENIZER(vocab_path or get_vocab_path(vocab_name), eos_token=eos_token)
