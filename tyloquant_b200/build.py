"""Build ``libmfqb200.so`` in-tree with nvcc for sm_100a.

``python tyloquant_b200/build.py`` (or ``build()``) compiles every source under
``csrc/`` into ``tyloquant_b200/lib/`` and links the shared library.  Objects are cached
by a hash of the source text, its headers and the flags, and translation units compile in
parallel.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB = os.path.join(LIBDIR, "libmfqb200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUFLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
           "-I", INCLUDE]
CUFLAGS += os.environ.get("MFQB_EXTRA_CUFLAGS", "").split()   # e.g. development-only -D switches
CXXFLAGS = ["-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unknown-pragmas", "-I", INCLUDE]


def _headers_digest() -> str:
    h = hashlib.sha256()
    for root in (CSRC, INCLUDE):
        for name in sorted(os.listdir(root)):
            if name.endswith((".h", ".cuh")):
                with open(os.path.join(root, name), "rb") as f:
                    h.update(name.encode())
                    h.update(f.read())
    return h.hexdigest()


def _compile(src: str, hdr_digest: str, verbose: bool) -> str:
    path = os.path.join(CSRC, src)
    is_cu = src.endswith(".cu")
    flags = CUFLAGS if is_cu else CXXFLAGS
    with open(path, "rb") as f:
        key = hashlib.sha256(f.read() + hdr_digest.encode() + " ".join(flags).encode()).hexdigest()[:16]
    obj = os.path.join(OBJDIR, f"{os.path.splitext(src)[0]}.{key}.o")
    if os.path.exists(obj):
        return obj
    for old in os.listdir(OBJDIR):
        if old.startswith(os.path.splitext(src)[0] + ".") and old.endswith(".o"):
            os.remove(os.path.join(OBJDIR, old))
    cmd = ([NVCC] + flags + (["-Xptxas", "-v"] if verbose else []) if is_cu else ["g++"] + flags) + ["-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        sys.stderr.write(r.stderr)
    return obj


def build(verbose: bool = False, jobs: int | None = None) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    sources = sorted(s for s in os.listdir(CSRC) if s.endswith((".cu", ".cpp")))
    digest = _headers_digest()
    with cf.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as pool:
        objs = list(pool.map(lambda s: _compile(s, digest, verbose), sources))
    stamp = hashlib.sha256(" ".join(sorted(objs)).encode()).hexdigest()
    stamp_file = os.path.join(LIBDIR, "link.stamp")
    if os.path.exists(LIB) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return LIB
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                  "-Xcompiler", "-fPIC", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"linking failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
