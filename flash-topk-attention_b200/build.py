"""Build libftk_sm100.so in-tree with nvcc for sm_100a.

    python flash-topk-attention_b200/build.py [--force]

Each csrc/*.cu is compiled to an object under build/ and the objects are
linked into lib/libftk_sm100.so (CUDA runtime linked statically; the driver
API is reached through cudaGetDriverEntryPoint, so the library also loads on
a machine without a GPU driver).
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libftk_sm100.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
    "-lineinfo", "-Xcompiler", "-fPIC",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return max(os.path.getmtime(h) for h in hs) if hs else 0.0


def _compile(src: str, force: bool) -> str:
    obj = os.path.join(OBJ, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    newest = max(os.path.getmtime(spath), _headers_mtime())
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj
    cmd = [NVCC, *FLAGS, "-c", spath, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force), srcs))
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= max(os.path.getmtime(o) for o in objs)):
        return LIB
    cmd = [NVCC, "-shared", "-o", LIB, *objs, "-gencode",
           "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


PROBE_SRC = os.path.join(os.path.dirname(HERE), "tests", "native", "wait_probe.cu")
PROBE_LIB = os.path.join(os.path.dirname(HERE), "tests", "native", "libftk_wait_probe.so")


def build_wait_probe(force: bool = False) -> str:
    """Test-only library: the bounded waits of csrc/ftk_sm100.cuh compiled with a
    wait limit of 200 000 clock ticks (tests/native/wait_probe.cu)."""
    if not os.path.exists(PROBE_SRC):
        return ""
    newest = max(os.path.getmtime(PROBE_SRC), _headers_mtime())
    if not force and os.path.exists(PROBE_LIB) and os.path.getmtime(PROBE_LIB) >= newest:
        return PROBE_LIB
    cmd = [NVCC, *FLAGS, "-DFTK_WAIT_CYCLES=200000LL", "-I", CSRC, "-shared", "-cudart", "static",
           PROBE_SRC, "-o", PROBE_LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for wait_probe.cu:\n{r.stdout}\n{r.stderr}")
    return PROBE_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    print(build_wait_probe(force="--force" in sys.argv))
