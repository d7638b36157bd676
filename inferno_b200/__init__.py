"""B200-native attention backend: paged GQA decode, causal prefill, absorbed-MLA decode and the
fused RoPE + KV-append that feeds them, as sm_100a CUDA kernels behind a C ABI."""
from .lib import InfernoError, load  # noqa: F401

__all__ = ["InfernoError", "load", "CudaBackend"]


def __getattr__(name):
    if name == "CudaBackend":
        from .backend import CudaBackend
        return CudaBackend
    raise AttributeError(name)
