"""Tokenizer throughput on the host: the native trie against the Python walk.

    python benchmarks/tokenizer_bench.py [--mb 4] [--threads 0]

Encodes the bundled ShareGPT sample repeated to ``--mb`` megabytes: one call on the whole text (ids returned as a
Python list), the same through the Python walk, and ``encode_batch`` over 20 kB pieces with list and with numpy
outputs.  Prints one JSON line; every variant is checked to give the same ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def best(fn, repeat: int = 3):
    out, t = None, float("inf")
    for _ in range(repeat):
        t0 = time.perf_counter()
        out = fn()
        t = min(t, time.perf_counter() - t0)
    return out, t


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=float, default=4.0)
    ap.add_argument("--threads", type=int, default=0)
    a = ap.parse_args()
    from rwkvtune_b200.data.tokenizers import get_tokenizer

    tok = get_tokenizer()
    sample = open(os.path.join(ROOT, "examples", "data", "sharegpt_sample.jsonl"), encoding="utf-8").read()
    text = sample * max(1, int(a.mb * 1e6 / len(sample.encode("utf-8"))))
    raw = text.encode("utf-8")
    mb = len(raw) / 1e6
    pieces = [text[i:i + 20000] for i in range(0, len(text), 20000)]
    rec = {"megabytes": round(mb, 2), "native": tok._native is not None, "cores": os.cpu_count()}
    py_ids, t_py = best(lambda: tok._encode_python(raw), 1)
    rec["python_walk_mb_s"] = round(mb / t_py, 1)
    if tok._native is not None:
        ids, t = best(lambda: tok.encode(text))
        assert ids == py_ids
        rec["native_encode_mb_s"] = round(mb / t, 1)
        lists, t = best(lambda: tok.encode_batch(pieces, a.threads))
        assert sum(lists, []) == sum((tok._encode_python(p.encode("utf-8")) for p in pieces), [])
        rec["native_batch_lists_mb_s"] = round(mb / t, 1)
        arrays, t = best(lambda: tok.encode_batch(pieces, a.threads, return_arrays=True))
        assert [x.tolist() for x in arrays] == lists
        rec["native_batch_arrays_mb_s"] = round(mb / t, 1)
        rec["tokens"] = len(ids)
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
