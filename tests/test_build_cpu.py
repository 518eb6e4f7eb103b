"""The ahead-of-time build script: what it compiles, how it decides that an object is current, its kernel table."""
import os
import shutil

import pytest

from rwkvtune_b200.csrc import build as B


def test_every_device_and_host_source_is_listed():
    srcs = B.sources()
    assert "gemm_tcgen05_2cta.cu" in srcs and "wkv7_tc.cu" in srcs and "zero_p2p.cu" in srcs
    assert "wkv7_cpu.cpp" in srcs and "tokenizer_trie.cu" in srcs
    assert srcs == sorted(srcs) and all(s.endswith((".cu", ".cpp")) for s in srcs)
    assert "-gencode" in B.ARCH_FLAGS and "arch=compute_100a,code=sm_100a" in B.ARCH_FLAGS       # sm_100a only
    assert "-lineinfo" in B.COMMON_FLAGS


def test_digest_follows_sources_headers_and_flags(tmp_path, monkeypatch):
    work = tmp_path / "csrc"
    work.mkdir()
    (work / "a.cu").write_text("// a\n")
    (work / "b.cpp").write_text("// b\n")
    (work / "common.cuh").write_text("// h1\n")
    monkeypatch.setattr(B, "HERE", str(work))
    assert B.sources() == ["a.cu", "b.cpp"]
    d_cu, d_cpp = B._digest(str(work / "a.cu")), B._digest(str(work / "b.cpp"))
    (work / "common.cuh").write_text("// h2\n")                  # a shared header changes every digest
    assert B._digest(str(work / "a.cu")) != d_cu and B._digest(str(work / "b.cpp")) != d_cpp
    d_cu = B._digest(str(work / "a.cu"))
    monkeypatch.setattr(B, "COMMON_FLAGS", B.COMMON_FLAGS + ["-DX"])      # device flags touch device sources only
    assert B._digest(str(work / "a.cu")) != d_cu
    d_cpp = B._digest(str(work / "b.cpp"))
    monkeypatch.setattr(B, "HOST_FLAGS", B.HOST_FLAGS + ["-DY"])
    assert B._digest(str(work / "b.cpp")) != d_cpp


def test_kernel_table_reads_the_compiler_report(tmp_path, monkeypatch):
    work = tmp_path / "csrc"
    (work / "build").mkdir(parents=True)
    (work / "k.cu").write_text("// k\n")
    (work / "build" / "k.ptxas.txt").write_text(
        "ptxas info    : 0 bytes gmem\n"
        "ptxas info    : Compiling entry function '_Z6kernelPf' for 'sm_100a'\n"
        "ptxas info    : Function properties for _Z6kernelPf\n"
        "    16 bytes stack frame, 8 bytes spill stores, 12 bytes spill loads\n"
        "ptxas info    : Used 40 registers, used 1 barriers, 256 bytes smem\n")
    monkeypatch.setattr(B, "HERE", str(work))
    table = B.ptxas_table()
    rows = table.splitlines()
    assert rows[0].startswith("| source | kernel | registers") and len(rows) == 3
    assert "`k.cu`" in rows[2] and "| 40 | 16 | 8 / 12 | 256 |" in rows[2]
    assert ("kernel" in rows[2]) and ("_Z6kernelPf" not in rows[2] or shutil.which("c++filt") is None)


@pytest.mark.skipif(shutil.which("g++") is None and shutil.which("c++") is None, reason="no host compiler")
def test_host_only_source_compiles_and_stale_objects_go(tmp_path, monkeypatch):
    work = tmp_path / "csrc"
    work.mkdir()
    (work / "h.cpp").write_text('extern "C" __attribute__((visibility("default"))) int answer() { return 42; }\n')
    monkeypatch.setattr(B, "HERE", str(work))
    obj = B._compile_one("h.cpp", verbose=False)
    assert os.path.exists(obj) and os.path.exists(obj + ".sha")
    stamp = os.path.getmtime(obj)
    assert B._compile_one("h.cpp", verbose=False) == obj and os.path.getmtime(obj) == stamp       # current: not rebuilt
    (work / "build" / "gone.o").write_text("")
    (work / "build" / "gone.o.sha").write_text("")
    (work / "h.cpp").write_text("this does not compile\n")
    with pytest.raises(RuntimeError, match="compilation failed for h.cpp"):
        B._compile_one("h.cpp", verbose=False)
