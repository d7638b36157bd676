"""Builds libinferno_attn.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m inferno_b200.build [--force] [--kprof]

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is installed.

--kprof builds a second, instrumented copy of the library into inferno_b200/kprof/ (compiled with
-DINF_KPROF: the tcgen05 kernels record a timeline of one CTA with %globaltimer and the host prints it to
stderr after each launch, synchronising to do so).  It is a diagnostic build, never the default; select it
with INFERNO_ATTN_LIB=inferno_b200/kprof/libinferno_attn.so.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libinferno_attn.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header() -> float:
    t = os.path.getmtime(os.path.join(HERE, "..", "include", "inferno_attn.h"))
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h")):
            t = max(t, os.path.getmtime(os.path.join(CSRC, f)))
    return t


def _compile(src: str, force: bool, out_dir: str = CSRC, extra=()) -> str:
    obj = os.path.join(out_dir, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(spath), _newest_header()):
        return obj
    log = subprocess.run([NVCC, *FLAGS, *extra, "-c", spath, "-o", obj], capture_output=True, text=True)
    with open(obj + ".log", "w") as f:
        f.write(log.stdout + log.stderr)
    if log.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{log.stdout}\n{log.stderr}")
    return obj


def build(force: bool = False, kprof: bool = False) -> str:
    srcs = sources()
    out_dir, lib, extra = CSRC, LIB, ()
    if kprof:
        out_dir = os.path.join(HERE, "kprof")
        os.makedirs(out_dir, exist_ok=True)
        lib, extra = os.path.join(out_dir, "libinferno_attn.so"), ("-DINF_KPROF",)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, out_dir, extra), srcs))
    if force or not os.path.exists(lib) or any(os.path.getmtime(o) > os.path.getmtime(lib) for o in objs):
        r = subprocess.run([NVCC, "-shared", "-o", lib, *objs, "-lcudart_static", "-ldl", "-lpthread", "-lrt",
                            "-Xlinker", "--no-undefined"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, kprof="--kprof" in sys.argv))
