"""Ahead-of-time build of the native library for sm_100a.

``python -m rwkvtune_b200.csrc.build`` compiles every ``*.cu`` in this directory with
``nvcc -gencode arch=compute_100a,code=sm_100a`` (and the host-only ``*.cpp`` files with the host compiler) and links them into
``librwkvtune_b200.so`` next to the sources.  The kernels depend on the CUDA runtime
only (no libtorch), so nvcc cross-compiles them on a machine without a GPU in a few
seconds per file.  The reference instead JIT-compiles its kernels on the user's
machine at first use (``rwkvtune/models/rwkv7/operators/wkv_loader.py:260-307``).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "librwkvtune_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
                "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def nvcc_path() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


HOST_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-fno-math-errno"]


def sources() -> List[str]:
    """Every ``*.cu`` (nvcc, sm_100a) and every ``*.cpp`` (host-only code, the host compiler) in this directory."""
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cu", ".cpp")))


def host_compiler() -> str:
    found = shutil.which(os.environ.get("CXX", "g++")) or shutil.which("c++")
    if not found:
        raise RuntimeError("no host C++ compiler found; set CXX")
    return found


def _digest(path: str) -> str:
    h = hashlib.sha256()
    for dep in [path] + sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cuh")):
        with open(dep, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(HOST_FLAGS if path.endswith(".cpp") else ARCH_FLAGS + COMMON_FLAGS).encode())
    return h.hexdigest()


DEBUG_LIB_NAME = "librwkvtune_b200_debug.so"
DEBUG_FLAGS = ["-DRWKV_DEBUG_BOUNDS"]


def _compile_one(src: str, verbose: bool, debug: bool = False) -> str:
    obj_dir = os.path.join(HERE, "build_debug" if debug else "build")
    os.makedirs(obj_dir, exist_ok=True)
    stem = os.path.splitext(src)[0]
    obj = os.path.join(obj_dir, stem + ".o")
    stamp = obj + ".sha"
    digest = _digest(os.path.join(HERE, src)) + ("-debug" if debug else "")
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest:
        return obj
    if src.endswith(".cpp"):
        cmd = [host_compiler()] + HOST_FLAGS + (DEBUG_FLAGS if debug else []) + ["-c", os.path.join(HERE, src), "-o", obj]
    else:
        cmd = ([nvcc_path()] + ARCH_FLAGS + COMMON_FLAGS + (DEBUG_FLAGS if debug else [])
               + ["-Xptxas", "-v", "-c", os.path.join(HERE, src), "-o", obj])
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compilation failed for {src}:\n{res.stdout}\n{res.stderr}")
    if src.endswith(".cu"):
        with open(os.path.join(obj_dir, stem + ".ptxas.txt"), "w") as fh:
            fh.write(res.stderr)
    if verbose:
        print(f"[build] {src} ok")
    with open(stamp, "w") as fh:
        fh.write(digest)
    return obj


def build(verbose: bool = True, force: bool = False, debug: bool = False) -> str:
    """Compile and link; returns the path of the shared library.  ``debug=True`` builds the bounds-recording variant
    (``librwkvtune_b200_debug.so``: data-dependent indices are range-checked, violations are recorded in a device
    word and skipped, nothing traps); ``RWKVTUNE_DEBUG_LIB=1`` makes the package load it."""
    if force:
        shutil.rmtree(os.path.join(HERE, "build_debug" if debug else "build"), ignore_errors=True)
    srcs = sources()
    obj_dir = os.path.join(HERE, "build_debug" if debug else "build")
    if os.path.isdir(obj_dir):      # objects of sources that no longer exist
        stems = {os.path.splitext(s)[0] for s in srcs}
        for f in os.listdir(obj_dir):
            if f.split(".")[0] not in stems:
                os.remove(os.path.join(obj_dir, f))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, verbose, debug), srcs))
    lib = os.path.join(HERE, DEBUG_LIB_NAME if debug else LIB_NAME)
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < newest:
        cmd = [nvcc_path(), "-shared", "-o", lib] + objs
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"[build] linked {lib}")
    return lib


def ptxas_table(debug: bool = False) -> str:
    """Markdown table of what ``ptxas -v`` reported for every kernel of the last build: registers, stack frame,
    spill stores / loads and static shared memory (dynamic shared memory is a launch parameter and not listed)."""
    import re

    obj_dir = os.path.join(HERE, "build_debug" if debug else "build")
    lines = ["| source | kernel | registers | stack frame (B) | spill stores / loads (B) | static shared memory (B) |",
             "|---|---|---|---|---|---|"]
    demangle = shutil.which("c++filt")
    for src in sources():
        path = os.path.join(obj_dir, os.path.splitext(src)[0] + ".ptxas.txt")
        if not src.endswith(".cu") or not os.path.exists(path):
            continue
        for block in re.split(r"ptxas info\s+: Compiling entry function '", open(path).read())[1:]:
            name = block.split("'")[0]
            if demangle:
                name = subprocess.run([demangle, name], capture_output=True, text=True).stdout.strip() or name
            name = re.sub(r"^void ", "", name.replace("(anonymous namespace)::", "").split("(")[0])
            regs = re.search(r"Used (\d+) registers", block)
            frame = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", block)
            smem = re.search(r"(\d+) bytes smem", block)
            lines.append(f"| `{src}` | `{name}` | {regs.group(1) if regs else '?'} | {frame.group(1) if frame else '?'} | "
                         f"{frame.group(2) if frame else '?'} / {frame.group(3) if frame else '?'} | "
                         f"{smem.group(1) if smem else 0} |")
    return "\n".join(lines)


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv, debug="--debug" in sys.argv)
    if "--ptxas" in sys.argv:
        print(ptxas_table(debug="--debug" in sys.argv))
