"""In-tree builder for the native libraries.

Two shared objects are produced under ``bloomery_b200/_C``:

* ``libbloomery_cuda.so`` -- every ``csrc/*.cu`` compiled for ``sm_100a`` only
  (``-gencode arch=compute_100a,code=sm_100a``); plain C ABI, loaded with ctypes.
* ``libbloomery_host.so`` -- ``csrc/host/*.cpp``: GGUF block decode oracle, CPU
  quantised dots (scalar mirror of the device units, AVX2 paths for Q4_K, Q6_K and Q8_0 rows and AVX-512 VNNI paths
  for Q4_K, Q5_K, Q6_K, Q8_0 and the int8 + f32-scale rows, picked at run time by CPU feature), the worker pool and the CPU expert leg.

nvcc cross-compiles without a GPU, so ``python -m bloomery_b200.build`` is also the
"does it build" check.  A content hash of sources and flags makes a rebuild a no-op.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
OUT = os.path.join(ROOT, "_C")
OBJ = os.path.join(OUT, "obj")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]
HOST_FLAGS = ["-std=c++17", "-O3", "-fPIC", "-mavx2", "-mfma", "-mf16c", "-pthread", "-fno-strict-aliasing"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")


def _hash(paths: List[str], flags: List[str]) -> str:
    h = hashlib.sha256()
    for f in flags:
        h.update(f.encode())
    deps = sorted(set(paths + [os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith((".cuh", ".h", ".hpp"))]
                      + [os.path.join(CSRC, "host", n) for n in os.listdir(os.path.join(CSRC, "host")) if n.endswith((".h", ".hpp"))]))
    for p in deps:
        h.update(p.encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + r.stdout)


def _build_lib(name: str, sources: List[str], compiler: str, flags: List[str], link: List[str], verbose: bool) -> str:
    os.makedirs(OBJ, exist_ok=True)
    lib = os.path.join(OUT, name)
    stamp = lib + ".hash"
    digest = _hash(sources, [compiler] + flags + link)
    if os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read() == digest:
        return lib
    objs = []

    def one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        _run([compiler] + flags + ["-I", CSRC, "-c", src, "-o", obj])
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(sources)))) as ex:
        objs = list(ex.map(one, sources))
    _run([compiler, "-shared", "-o", lib] + objs + link)
    with open(stamp, "w") as fh:
        fh.write(digest)
    if verbose:
        print(f"built {lib}", file=sys.stderr)
    return lib


def source_hash() -> str:
    """Digest of the sources and flags the loaded CUDA library was built from (keys the cost store)."""
    stamp = os.path.join(OUT, "libbloomery_cuda.so.hash")
    try:
        return open(stamp).read().strip()[:16]
    except OSError:
        return "unbuilt"


def build_cuda(verbose: bool = False) -> str:
    srcs = sorted(os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith(".cu"))
    inc = []
    return _build_lib("libbloomery_cuda.so", srcs, _nvcc(), NVCC_FLAGS + inc, [], verbose)


def build_host(verbose: bool = False) -> str:
    hdir = os.path.join(CSRC, "host")
    srcs = sorted(os.path.join(hdir, n) for n in os.listdir(hdir) if n.endswith(".cpp"))
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    return _build_lib("libbloomery_host.so", srcs, cxx, HOST_FLAGS, ["-pthread"], verbose)


def build_all(verbose: bool = False) -> None:
    build_host(verbose)
    build_cuda(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
