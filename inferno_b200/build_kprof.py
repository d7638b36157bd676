"""Builds an instrumented copy of the library (-DINF_KPROF: in-kernel cycle accounting printed to stderr)
into inferno_b200/kprof/libinferno_attn.so.  Select it with INFERNO_ATTN_LIB; it is never the default."""
import os
import subprocess

from . import build as B

OUT = os.path.join(B.HERE, "kprof")


def build():
    os.makedirs(OUT, exist_ok=True)
    objs = []
    procs = []
    for src in B.sources():
        obj = os.path.join(OUT, src[:-3] + ".o")
        objs.append(obj)
        procs.append(subprocess.Popen([B.NVCC, *[f for f in B.FLAGS if f not in ("-Xptxas", "-v")], "-DINF_KPROF", "-c",
                                       os.path.join(B.CSRC, src), "-o", obj]))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed")
    lib = os.path.join(OUT, "libinferno_attn.so")
    subprocess.check_call([B.NVCC, "-shared", "-o", lib, *objs, "-lcudart_static", "-ldl", "-lpthread", "-lrt"])
    return lib


if __name__ == "__main__":
    print(build())
