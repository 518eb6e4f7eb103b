"""HF-style tokenizer facade over :class:`TRIE_TOKENIZER`.

Same public methods and the same ``tokenizer_config.json`` layout as
``rwkvtune/data/tokenizers/auto_tokenizer.py:12-787``: ``encode`` / ``decode(skip_special_tokens)``,
``__call__(return_tensors="pt")``, ``apply_chat_template``, ``batch_decode``,
``add_special_tokens`` (extends the vocabulary), ``add_special_token_with_id`` (re-maps an id, e.g.
``<|im_end|>`` -> 0), ``from_pretrained`` / ``save_pretrained``.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Any, Dict, List, Optional, Sequence, Union

from .rwkv_tokenizer import TRIE_TOKENIZER
from .special_token_handler import SpecialTokenTrie

TOKENIZER_CONFIG_NAME = "tokenizer_config.json"
VOCAB_CANDIDATES = ("vocab.txt", "rwkv_vocab_v20230424.txt")
_ROLE_KEYS = ("eos_token", "pad_token", "bos_token", "unk_token")


class TokenizerConfig:
    _FIELDS = ("tokenizer_class", "vocab_file", "model_max_length", "bos_token", "eos_token", "pad_token",
               "unk_token", "add_bos_token", "add_eos_token", "clean_up_tokenization_spaces", "chat_template")

    def __init__(self, tokenizer_class: str = "RWKV_TOKENIZER", vocab_file: Optional[str] = None,
                 model_max_length: int = 4096, bos_token: Optional[str] = None, eos_token: str = "\n\n",
                 pad_token: Optional[str] = None, unk_token: Optional[str] = None, add_bos_token: bool = False,
                 add_eos_token: bool = False, clean_up_tokenization_spaces: bool = False,
                 chat_template: Optional[str] = None, **kwargs: Any):
        self.tokenizer_class = tokenizer_class
        self.vocab_file = vocab_file
        self.model_max_length = model_max_length
        self.bos_token, self.eos_token, self.pad_token, self.unk_token = bos_token, eos_token, pad_token, unk_token
        self.add_bos_token, self.add_eos_token = add_bos_token, add_eos_token
        self.clean_up_tokenization_spaces = clean_up_tokenization_spaces
        self.chat_template = chat_template
        self._extra_config = kwargs

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "TokenizerConfig":
        return cls(**config_dict)

    @classmethod
    def from_json_file(cls, json_file: str) -> "TokenizerConfig":
        with open(json_file, "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    def to_dict(self) -> Dict[str, Any]:
        d = {k: getattr(self, k) for k in self._FIELDS}
        d.update(self._extra_config)
        return {k: v for k, v in d.items() if v is not None}

    def to_json_file(self, json_file: str) -> None:
        os.makedirs(os.path.dirname(json_file) or ".", exist_ok=True)
        with open(json_file, "w", encoding="utf-8") as fh:
            json.dump(self.to_dict(), fh, indent=2, ensure_ascii=False)

    def save_pretrained(self, save_directory: str) -> None:
        self.to_json_file(os.path.join(save_directory, TOKENIZER_CONFIG_NAME))


class BatchEncoding(dict):
    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError as exc:
            raise AttributeError(name) from exc

    def to(self, device):
        for k, v in list(self.items()):
            if hasattr(v, "to"):
                self[k] = v.to(device)
        return self


class RWKVTokenizer(TRIE_TOKENIZER):
    def __init__(self, vocab_file: str, eos_token: Optional[Union[str, int]] = None, bos_token: Optional[str] = None,
                 pad_token: Optional[str] = None, unk_token: Optional[str] = None, add_bos_token: bool = False,
                 add_eos_token: bool = False, model_max_length: int = 4096, chat_template: Optional[str] = None,
                 **kwargs: Any):
        self.additional_special_tokens: Dict[str, int] = {}
        self.additional_special_tokens_ids: List[int] = []
        self._special_token_trie = SpecialTokenTrie()
        self._extra_tokens: Dict[bytes, int] = {}
        super().__init__(vocab_file, eos_token=eos_token)
        self.vocab_file = vocab_file
        self.eos_token = eos_token if eos_token is not None else "\n\n"
        self.bos_token, self.pad_token, self.unk_token = bos_token, pad_token, unk_token
        self.add_bos_token, self.add_eos_token = add_bos_token, add_eos_token
        self.model_max_length = model_max_length
        self.chat_template = chat_template
        self.bos_token_id = self._get_token_id(bos_token) if bos_token else None
        self.pad_token_id = self._get_token_id(pad_token) if pad_token else self.eos_token_id
        self.unk_token_id = self._get_token_id(unk_token) if unk_token else None

    # ------------------------------------------------------------------ vocabulary edits
    def _get_token_id(self, token: Union[str, int, None]) -> Optional[int]:
        if isinstance(token, int):
            return token if token in self.idx2token else None
        if isinstance(token, str):
            if token in self.additional_special_tokens:
                return self.additional_special_tokens[token]
            return self.token2idx.get(token.encode("utf-8"))
        return None

    def _register(self, token: str, token_id: int) -> None:
        tb = token.encode("utf-8")
        old = self.idx2token.get(token_id)
        if old is not None and old != tb:
            self.token2idx.pop(old, None)
        prev_id = self.token2idx.get(tb)
        if prev_id is not None and prev_id != token_id:
            self.idx2token.pop(prev_id, None)
        self.idx2token[token_id] = tb
        self.token2idx[tb] = token_id
        self._insert(tb, token_id)
        self._extra_tokens[tb] = token_id
        self.vocab_size = max(self.vocab_size, token_id + 1)

    def _set_role(self, role: str, token: Optional[str], token_id: Optional[int]) -> None:
        if role in _ROLE_KEYS:
            if token is not None:
                setattr(self, role, token)
            setattr(self, role + "_id", token_id)

    def add_special_token_with_id(self, token: str, token_id: int, set_as: Optional[str] = None) -> bool:
        self._register(token, token_id)
        self.additional_special_tokens[token] = token_id
        if token_id not in self.additional_special_tokens_ids:
            self.additional_special_tokens_ids.append(token_id)
        self._special_token_trie.add(token)
        if set_as:
            self._set_role(set_as, token, token_id)
        return True

    def add_special_tokens(self, special_tokens_dict: Dict[str, Any], replace_additional_special_tokens: bool = False) -> int:
        added = 0
        if "additional_special_tokens" in special_tokens_dict:
            if replace_additional_special_tokens:
                self.additional_special_tokens, self.additional_special_tokens_ids = {}, []
            for token in special_tokens_dict["additional_special_tokens"]:
                if token in self.additional_special_tokens:
                    continue
                tid = self.token2idx.get(token.encode("utf-8"))
                if tid is None:
                    tid = self.vocab_size
                    self._register(token, tid)
                    added += 1
                self.additional_special_tokens[token] = tid
                if tid not in self.additional_special_tokens_ids:
                    self.additional_special_tokens_ids.append(tid)
                self._special_token_trie.add(token)
        for key, value in special_tokens_dict.items():
            if key == "additional_special_tokens":
                continue
            if isinstance(value, str):
                tid = self._get_token_id(value)
                if tid is None:
                    tid = self.vocab_size
                    self._register(value, tid)
                    self._special_token_trie.add(value)
                    added += 1
                self._set_role(key, value, tid)
            elif isinstance(value, int):
                self._set_role(key, None, value)
        return added

    def get_added_vocab(self) -> Dict[str, int]:
        return dict(self.additional_special_tokens)

    def __len__(self) -> int:
        return self.vocab_size

    # ------------------------------------------------------------------ text <-> ids
    def encode(self, text: str, add_special_tokens: bool = True, **kwargs: Any) -> List[int]:
        ids: List[int] = []
        if len(self._special_token_trie):
            for piece in self._special_token_trie.split(text):
                if piece in self.additional_special_tokens:
                    ids.append(self.additional_special_tokens[piece])
                else:
                    ids.extend(self.encodeBytes(piece.encode("utf-8")))
        else:
            ids = self.encodeBytes(text.encode("utf-8"))
        if add_special_tokens:
            if self.add_bos_token and self.bos_token_id is not None:
                ids = [self.bos_token_id] + ids
            if self.add_eos_token and self.eos_token_id is not None:
                ids = ids + [self.eos_token_id]
        return ids

    def encode_batch(self, texts: Sequence[str], num_threads: int = 0, return_arrays: bool = False,
                     add_special_tokens: bool = True):
        """:meth:`encode` of every text.  Plain configurations go to the native batch call; with registered special
        tokens or BOS / EOS insertion every text takes the :meth:`encode` route, so the ids are the same either way."""
        plain = not len(self._special_token_trie) and not (add_special_tokens and (self.add_bos_token or self.add_eos_token))
        if plain:
            return super().encode_batch(texts, num_threads, return_arrays)
        out = [self.encode(t, add_special_tokens=add_special_tokens) for t in texts]
        if return_arrays:
            import numpy as np

            return [np.asarray(o, dtype=np.int32) for o in out]
        return out

    def decode(self, token_ids, skip_special_tokens: bool = False, **kwargs: Any) -> str:
        if hasattr(token_ids, "tolist"):
            token_ids = token_ids.tolist()
        if isinstance(token_ids, int):
            token_ids = [token_ids]
        if skip_special_tokens:
            drop = set(self.additional_special_tokens_ids)
            for tid, tok in ((self.eos_token_id, self.eos_token), (self.pad_token_id, self.pad_token),
                             (self.bos_token_id, self.bos_token)):
                if tid is not None and isinstance(tok, str) and tok in self.additional_special_tokens:
                    drop.add(tid)
            token_ids = [t for t in token_ids if int(t) not in drop]
        return super().decode(token_ids)

    def batch_decode(self, sequences, skip_special_tokens: bool = False, **kwargs: Any) -> List[str]:
        if hasattr(sequences, "tolist"):
            sequences = sequences.tolist()
        return [self.decode(s, skip_special_tokens=skip_special_tokens) for s in sequences]

    def __call__(self, text: Union[str, Sequence[str]], return_tensors: Optional[str] = None, padding: bool = True,
                 **kwargs: Any):
        single = isinstance(text, str)
        texts = [text] if single else list(text)
        seqs = self.encode_batch(texts) if len(texts) > 1 else [self.encode(texts[0])]
        if return_tensors == "pt":
            import torch

            width = max(len(s) for s in seqs)
            pad = self.pad_token_id if self.pad_token_id is not None else 0
            ids = torch.full((len(seqs), width), pad, dtype=torch.long)
            mask = torch.zeros((len(seqs), width), dtype=torch.long)
            for i, s in enumerate(seqs):
                ids[i, :len(s)] = torch.tensor(s, dtype=torch.long)
                mask[i, :len(s)] = 1
            return BatchEncoding({"input_ids": ids, "attention_mask": mask})
        if single:
            return BatchEncoding({"input_ids": seqs[0], "attention_mask": [1] * len(seqs[0])})
        return BatchEncoding({"input_ids": seqs, "attention_mask": [[1] * len(s) for s in seqs]})

    # ------------------------------------------------------------------ chat
    def _simple_format(self, messages: list, add_generation_prompt: bool = False) -> str:
        names = {"system": "System", "user": "User", "assistant": "Assistant"}
        text = "".join(f"{names[m['role']]}: {m['content']}\n\n" for m in messages if m.get("role") in names)
        return text + ("Assistant:" if add_generation_prompt else "")

    def apply_chat_template(self, messages: list, tokenize: bool = False, add_generation_prompt: bool = False,
                            chat_template: Optional[str] = None, **kwargs: Any):
        template = chat_template or self.chat_template
        if template:
            from jinja2 import Template

            text = Template(template).render(messages=messages, add_generation_prompt=add_generation_prompt,
                                             eos_token=self.eos_token, bos_token=self.bos_token or "", **kwargs)
        else:
            text = self._simple_format(messages, add_generation_prompt)
        return self.encode(text) if tokenize else text

    # ------------------------------------------------------------------ persistence
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, **kwargs: Any) -> "RWKVTokenizer":
        d = pretrained_model_name_or_path
        if not os.path.isdir(d):
            raise ValueError(f"directory does not exist: {d}")
        cfg_file = os.path.join(d, TOKENIZER_CONFIG_NAME)
        cfg = TokenizerConfig.from_json_file(cfg_file) if os.path.exists(cfg_file) else TokenizerConfig()
        vocab = next((os.path.join(d, n) for n in VOCAB_CANDIDATES if os.path.exists(os.path.join(d, n))), None)
        if vocab is None:
            raise FileNotFoundError(f"no vocabulary file ({' / '.join(VOCAB_CANDIDATES)}) in {d}")
        template = cfg.chat_template
        tfile = os.path.join(d, "chat_template.jinja")
        if template is None and os.path.exists(tfile):
            with open(tfile, "r", encoding="utf-8") as fh:
                template = fh.read()
        init = dict(vocab_file=vocab, eos_token=cfg.eos_token, bos_token=cfg.bos_token, pad_token=cfg.pad_token,
                    unk_token=cfg.unk_token, add_bos_token=cfg.add_bos_token, add_eos_token=cfg.add_eos_token,
                    model_max_length=cfg.model_max_length, chat_template=template)
        init.update(kwargs)
        tok = cls(**init)
        extra = cfg._extra_config.get("additional_special_tokens") or []
        if extra and isinstance(extra[0], dict):
            for item in extra:
                if "id" in item:
                    tok.add_special_token_with_id(item["token"], int(item["id"]))
                elif "ids" in item and len(item["ids"]) == 1:
                    tok.add_special_token_with_id(item["token"], int(item["ids"][0]))
                else:
                    tok.add_special_tokens({"additional_special_tokens": [item["token"]]})
        elif extra:
            ids = cfg._extra_config.get("additional_special_tokens_ids", [])
            for i, token in enumerate(extra):
                if i < len(ids):
                    tok.add_special_token_with_id(token, int(ids[i]))
                else:
                    tok.add_special_tokens({"additional_special_tokens": [token]})
        for role in _ROLE_KEYS:
            text = getattr(tok, role, None)
            if isinstance(text, str):
                ids = tok.encode(text, add_special_tokens=False)
                setattr(tok, role + "_id", ids[0] if ids else None)
        if tok.pad_token is None:
            tok.pad_token_id = tok.eos_token_id
        return tok

    def save_pretrained(self, save_directory: str) -> None:
        os.makedirs(save_directory, exist_ok=True)
        cfg = TokenizerConfig(vocab_file="vocab.txt", model_max_length=self.model_max_length, bos_token=self.bos_token,
                              eos_token=self.eos_token if isinstance(self.eos_token, str) else None,
                              pad_token=self.pad_token, unk_token=self.unk_token, add_bos_token=self.add_bos_token,
                              add_eos_token=self.add_eos_token, chat_template=self.chat_template)
        if self.additional_special_tokens:
            cfg._extra_config["additional_special_tokens"] = [
                {"token": t, "id": i} for t, i in self.additional_special_tokens.items()]
        cfg.save_pretrained(save_directory)
        target = os.path.join(save_directory, "vocab.txt")
        if os.path.abspath(self.vocab_file) != os.path.abspath(target):
            shutil.copyfile(self.vocab_file, target)
        if self.chat_template:
            with open(os.path.join(save_directory, "chat_template.jinja"), "w", encoding="utf-8") as fh:
                fh.write(self.chat_template)


class AutoTokenizer:
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str, **kwargs: Any) -> RWKVTokenizer:
        d = pretrained_model_name_or_path
        cfg_file = os.path.join(d, TOKENIZER_CONFIG_NAME)
        if os.path.exists(cfg_file):
            kind = TokenizerConfig.from_json_file(cfg_file).tokenizer_class
            if kind not in ("RWKV_TOKENIZER", "RWKVTokenizer", "TRIE_TOKENIZER"):
                raise ValueError(f"unsupported tokenizer_class {kind!r}")
        return RWKVTokenizer.from_pretrained(d, **kwargs)
