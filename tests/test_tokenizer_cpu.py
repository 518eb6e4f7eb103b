"""Tokenizer behaviour on CPU: round trips over the shipped vocabulary, special tokens, chat templates, ChatML
set-up, files on disk, pickling, and the text-level special-token helpers."""
import json
import os
import pickle

import pytest
import torch

from rwkvtune_b200.data.tokenizers import AutoTokenizer, RWKVTokenizer, get_tokenizer, get_vocab_path
from rwkvtune_b200.data.tokenizers import chatml_utils
from rwkvtune_b200.data.tokenizers.special_token_handler import (SpecialTokenTrie, decode_with_special_tokens,
                                                                 encode_with_special_tokens)


@pytest.fixture(scope="module")
def base():
    return get_tokenizer()


def _fresh():
    return RWKVTokenizer(get_vocab_path())


@pytest.mark.parametrize("text", ["Hello, world!", "多语言 テキスト 한국어 🙂🚀", "tabs\tand\nnewlines\n\nUser: hi", "\x00\x01 raw",
                                  "a" * 300 + " " * 17, ""])
def test_round_trip_and_greedy_longest_match(base, text):
    ids = base.encode(text)
    assert base.decode(ids) == text
    assert all(0 < i < 65530 for i in ids)
    if text:
        # greedy longest match: no two neighbouring tokens whose concatenation is itself the longest match at that point
        first = base.idx2token[ids[0]]
        longer = [t for t in (text.encode("utf-8")[:len(first) + k] for k in range(1, 4)) if len(t) > len(first)]
        assert not any(t in base.token2idx for t in longer)


def test_eos_is_the_double_newline_and_bytes_decode_tolerantly(base):
    assert base.eos_token_id == 261 and base.encode("\n\n") == [261]
    euro = "€".encode("utf-8")
    ids = [base.token2idx[euro[:1]], base.token2idx[euro[1:2]]]        # a character cut in the middle
    out = base.decode(ids)
    assert isinstance(out, str)                                          # no exception, replacement character or partial
    assert base.decode(ids + [base.token2idx[euro[2:3]]]) == "€"


def test_special_tokens_get_reserved_ids_and_split_the_text():
    tok = _fresh()
    assert tok.pad_token_id == tok.eos_token_id == 261 and len(tok) == 65530
    assert tok.add_special_tokens({"additional_special_tokens": ["<|im_start|>", "<|im_end|>"]}) == 2
    assert tok.add_special_tokens({"additional_special_tokens": ["<|im_start|>"]}) == 0       # already there
    a, b = tok.additional_special_tokens["<|im_start|>"], tok.additional_special_tokens["<|im_end|>"]
    assert (a, b) == (65530, 65531) and len(tok) == 65532 and tok.get_added_vocab()["<|im_end|>"] == b
    ids = tok.encode("<|im_start|>user\nhi<|im_end|>")
    assert ids[0] == a and ids[-1] == b and a not in ids[1:-1]
    assert tok.decode(ids) == "<|im_start|>user\nhi<|im_end|>"
    assert tok.decode(ids, skip_special_tokens=True) == "user\nhi"
    assert tok.batch_decode([ids, ids[1:-1]], skip_special_tokens=True) == ["user\nhi", "user\nhi"]
    # a token planted on an existing id takes that id over and can become a role token
    assert tok.add_special_token_with_id("<|stop|>", 0, set_as="eos_token")
    assert tok.eos_token == "<|stop|>" and tok.eos_token_id == 0 and tok.encode("x<|stop|>")[-1] == 0


def test_call_pads_and_returns_tensors():
    tok = _fresh()
    out = tok(["a", "hello world"], return_tensors="pt")
    assert out["input_ids"].shape == out["attention_mask"].shape == (2, 2)
    assert out["attention_mask"].tolist() == [[1, 0], [1, 1]] and out["input_ids"][0, 1] == tok.pad_token_id
    single = tok("hello world")
    assert single["input_ids"] == tok.encode("hello world")
    assert isinstance(tok("hi", return_tensors="pt")["input_ids"], torch.Tensor)


def test_default_and_chatml_templates():
    tok = _fresh()
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]
    plain = tok.apply_chat_template(msgs[:1], tokenize=False, add_generation_prompt=True)
    assert plain == "User: hi\n\nAssistant:"
    assert tok.apply_chat_template(msgs[:1], tokenize=True, add_generation_prompt=True) == tok.encode(plain)
    res = chatml_utils.setup_chatml_tokenizer(tok)
    assert res["success"] and res["template_set"] and not res["errors"]
    ok, errors = chatml_utils.validate_chatml_tokenizer(tok)
    assert ok and errors == []
    assert tok.eos_token == "<|im_end|>" and tok.eos_token_id == 0          # re-mapped to the unused id 0
    text = tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
    assert text.count("<|im_start|>") == 3 and text.count("<|im_end|>") == 2 and text.endswith("<|im_start|>assistant\n")
    ids = tok.encode(text)
    assert ids.count(tok.additional_special_tokens["<|im_start|>"]) == 3 and ids.count(0) == 2
    good, diag = chatml_utils.verify_chatml_formatting(tok)
    assert good and diag["num_tokens"] > 0 and not diag["errors"]
    bare = _fresh()
    assert chatml_utils.validate_chatml_tokenizer(bare) == (False, ["tokenizer.chat_template is not set"])


def test_save_and_reload_keep_special_tokens_and_template(tmp_path):
    tok = _fresh()
    chatml_utils.setup_chatml_tokenizer(tok)
    tok.save_pretrained(str(tmp_path))
    assert {"vocab.txt", "tokenizer_config.json"} <= set(os.listdir(tmp_path))
    cfg = json.load(open(tmp_path / "tokenizer_config.json"))
    assert cfg["eos_token"] == "<|im_end|>" and "<|im_start|>" in json.dumps(cfg)
    again = AutoTokenizer.from_pretrained(str(tmp_path))
    sample = "<|im_start|>user\n你好<|im_end|>\n"
    assert again.encode(sample) == tok.encode(sample) and again.eos_token_id == tok.eos_token_id == 0
    assert again.chat_template == tok.chat_template
    assert again.decode(again.encode(sample)) == sample


def test_tokenizers_survive_pickling(base):
    tok = _fresh()
    tok.add_special_tokens({"additional_special_tokens": ["<|tool|>"]})
    for t in (base, tok):
        clone = pickle.loads(pickle.dumps(t))
        s = "abc <|tool|> 数据"
        assert clone.encode(s) == t.encode(s) and clone.decode(t.encode(s)) == s


def test_text_level_helpers_accept_ids_and_id_sequences(base):
    mapping = {"<|a|>": 65530, "<|think|>": [65531, 65532], "<|a|><": 65533}      # the longest special token wins
    ids = encode_with_special_tokens("x<|a|>-<|think|>y<|a|><z", base, mapping)
    assert ids == (base.encode("x") + [65530] + base.encode("-") + [65531, 65532] + base.encode("y") + [65533]
                   + base.encode("z"))
    assert encode_with_special_tokens("plain", base.encode, {}) == base.encode("plain")
    back = decode_with_special_tokens(ids, base, mapping)
    assert back == "x<|a|>-<|think|>y<|a|><z"
    assert decode_with_special_tokens(ids, base.decode, mapping, skip_special_tokens=True) == "x-yz"
    # a character split over several byte tokens between two special tokens is decoded as one run
    euro = [base.token2idx[bytes([b])] for b in "€".encode("utf-8")]
    assert decode_with_special_tokens([65530] + euro + [65530], base, mapping) == "<|a|>€<|a|>"
    trie = SpecialTokenTrie()
    for t in mapping:
        trie.add(t)
    assert trie.split("<|a|>x<|a|><") == ["<|a|>", "x", "<|a|><"] and trie.split("") == [] and len(trie) == 3


def _native_or_skip(tok):
    if getattr(tok, "_native", None) is None:
        pytest.skip("native library not built")
    return tok


def test_native_trie_agrees_with_the_python_walk_on_text_and_raw_bytes(base):
    import random

    tok = _native_or_skip(base)
    rng = random.Random(0)
    alphabet = "abc XYZ,.\n\t的是不了人我在有他这為なにをはが한국어éüß🙂🚀"
    samples = ["".join(rng.choice(alphabet) for _ in range(rng.randint(0, 400))) for _ in range(60)]
    for s in samples:
        b = s.encode("utf-8")
        assert tok.encodeBytes(b) == tok._encode_python(b)
    for _ in range(40):                                   # arbitrary bytes, including invalid UTF-8
        b = bytes(rng.randrange(256) for _ in range(rng.randint(1, 300)))
        ids = tok.encodeBytes(b)
        assert ids == tok._encode_python(b) and tok.decodeBytes(ids) == b
    assert tok.encodeBytes(b"") == []


def test_native_batch_encoding_lists_arrays_and_threads(base):
    import numpy as np

    tok = _native_or_skip(base)
    texts = ["", "hello world", "多语言 🙂" * 50, "x" * 1000, "\n\n"] * 7
    want = [tok._encode_python(t.encode("utf-8")) for t in texts]
    for threads in (1, 3, 0):
        assert tok.encode_batch(texts, num_threads=threads) == want
    arrays = tok.encode_batch(texts, return_arrays=True)
    assert all(isinstance(a, np.ndarray) and a.dtype == np.int32 for a in arrays) and [a.tolist() for a in arrays] == want
    assert tok.encode_batch([]) == []


def test_native_trie_sees_tokens_added_later_and_survives_pickling():
    tok = _native_or_skip(_fresh())
    tok.add_special_tokens({"additional_special_tokens": ["<|late|>"]})
    late = tok.additional_special_tokens["<|late|>"]
    # the raw byte path too: the new token is part of the trie, not only of the text-level splitter
    assert tok.encodeBytes("a<|late|>b".encode()) == tok._encode_python("a<|late|>b".encode())
    assert late in tok.encodeBytes("a<|late|>b".encode())
    clone = pickle.loads(pickle.dumps(tok))
    assert clone._native is not None and clone._native is not tok._native
    assert clone.encodeBytes("a<|late|>b".encode()) == tok.encodeBytes("a<|late|>b".encode())


def test_python_fallback_is_complete_and_reports_uncovered_bytes(tmp_path, monkeypatch):
    from rwkvtune_b200.data.tokenizers import rwkv_tokenizer as mod

    vocab = tmp_path / "tiny_vocab.txt"
    vocab.write_text("1 'a' 1\n2 'b' 1\n3 'ab' 2\n4 'abc' 3\n5 b'\\xff' 1\n")
    for native in (True, False):
        monkeypatch.setattr(mod._NativeTrie, "_tried", not native)
        monkeypatch.setattr(mod._NativeTrie, "_lib", None)
        tok = mod.TRIE_TOKENIZER(str(vocab), eos_token="a")
        if not native:
            assert tok._native is None and tok._next is not None
        assert tok.encode("abab") == [3, 3] and tok.encode("abca") == [4, 1] and tok.encodeBytes(b"a\xffb") == [1, 5, 2]
        assert tok.encode_batch(["ab", "ba"]) == [[3], [2, 1]]
        with pytest.raises(ValueError, match="offset 2"):
            tok.encode("abz")
        with pytest.raises(ValueError, match="text 1"):
            tok.encode_batch(["ab", "zz"])
    monkeypatch.setattr(mod._NativeTrie, "_tried", False)


def test_batch_encoding_of_the_full_tokenizer_matches_encode_in_every_configuration():
    texts = ["hello <|im_start|>user", "plain text", "<|im_end|>", ""]
    plain = _fresh()
    assert plain.encode_batch(texts) == [plain.encode(t) for t in texts]
    assert plain(texts)["input_ids"] == [plain.encode(t) for t in texts]
    special = _fresh()
    special.add_special_tokens({"additional_special_tokens": ["<|im_start|>", "<|im_end|>"]})
    assert special.encode_batch(texts) == [special.encode(t) for t in texts]
    assert special.encode_batch(texts)[2] == [special.additional_special_tokens["<|im_end|>"]]
    framed = RWKVTokenizer(get_vocab_path(), add_eos_token=True)
    assert framed.encode_batch(texts) == [framed.encode(t) for t in texts] and framed.encode_batch(texts)[1][-1] == 261
    assert framed.encode_batch(texts, add_special_tokens=False) == [framed.encode(t, add_special_tokens=False) for t in texts]
    arrays = special.encode_batch(texts, return_arrays=True)
    assert [a.tolist() for a in arrays] == special.encode_batch(texts)
