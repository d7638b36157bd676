"""ctypes binding of libinferno_attn.so: one Python function per C-ABI entry point.

The library is the product; there is no Python or CPU fallback.  Importing this module
without the built library raises, and so does creating a context without a B200.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("INFERNO_ATTN_LIB") or os.path.join(_HERE, "libinferno_attn.so")  # env: an alternative build

INF_OK = 0
INF_UNSUPPORTED = 1
INF_E_BACKEND, INF_E_SHAPE, INF_E_CONFIG, INF_E_CACHE, INF_E_DTYPE, INF_E_ARG = -1, -2, -3, -4, -5, -6
DTYPE_F32, DTYPE_F16 = 0, 1
GQA_DECODE_STATIC_SCRATCH_BYTES = 32 << 20
MAX_PEERS, PEER_HANDLE_BYTES = 7, 72

ERROR_NAMES = {INF_E_BACKEND: "Backend", INF_E_SHAPE: "ShapeMismatch", INF_E_CONFIG: "Config", INF_E_CACHE: "Cache",
               INF_E_DTYPE: "DType", INF_E_ARG: "Argument"}


class InfernoError(RuntimeError):
    """An INF_E_* status; `.code` is the status, `.kind` mirrors the reference's Error variant."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.kind = ERROR_NAMES.get(code, str(code))


class RopeTable(C.Structure):
    _fields_ = [("inv_freq", C.c_void_p), ("rotary_dim", C.c_int32), ("attention_factor", C.c_float)]


class KvPool(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("num_pages", C.c_int32), ("page_size", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32)]


class KvPoolFp8(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("num_pages", C.c_int32), ("page_size", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("key_scale", C.c_float), ("value_scale", C.c_float)]


class MlaPool(C.Structure):
    _fields_ = [("rows", C.c_void_p), ("num_pages", C.c_int32), ("page_size", C.c_int32), ("latent_dim", C.c_int32),
                ("rope_dim", C.c_int32)]


class PageTable(C.Structure):
    _fields_ = [("pages", C.c_void_p), ("lens", C.c_void_p), ("batch", C.c_int32), ("max_pages", C.c_int32),
                ("host_pages", C.c_void_p), ("host_lens", C.c_void_p)]


_P = C.c_void_p
_I = C.c_int32
_F = C.c_float
_L = C.c_int64

# name -> (restype, argtypes); the list is also what the symbol-export test checks against the header
SIGNATURES = {
    "inf_ctx_create": (_I, [_I, _P, C.POINTER(_P)]),
    "inf_ctx_destroy": (_I, [_P]),
    "inf_ctx_set_stream": (_I, [_P, _P]),
    "inf_last_error": (C.c_char_p, [_P]),
    "inf_device_values_supported": (_I, [_P]),
    "inf_flush": (_I, [_P]),
    "inf_submit": (_I, [_P]),
    "inf_debug_drop_next_load": (_I, [_P, _I]),
    "inf_profile_enable": (_I, [_P, _I]),
    "inf_profile_read": (_I, [_P, C.c_char_p, C.POINTER(C.c_double), C.POINTER(_I)]),
    "inf_alloc": (_I, [_P, C.c_size_t, C.POINTER(_P)]),
    "inf_free": (_I, [_P, _P]),
    "inf_upload": (_I, [_P, _P, _P, C.c_size_t]),
    "inf_upload_f32_as_f16": (_I, [_P, _P, _P, C.c_size_t]),
    "inf_download": (_I, [_P, _P, _P, C.c_size_t]),
    "inf_copy": (_I, [_P, _P, _P, C.c_size_t]),
    "inf_memset_zero": (_I, [_P, _P, C.c_size_t]),
    "inf_rope_table_create": (_I, [_P, _P, _I, _I, _F, C.POINTER(RopeTable)]),
    "inf_rope_table_destroy": (_I, [_P, C.POINTER(RopeTable)]),
    "inf_kv_pool_create": (_I, [_P, _I, _I, _I, _I, C.POINTER(KvPool)]),
    "inf_kv_pool_destroy": (_I, [_P, C.POINTER(KvPool)]),
    "inf_mla_pool_create": (_I, [_P, _I, _I, _I, _I, C.POINTER(MlaPool)]),
    "inf_mla_pool_destroy": (_I, [_P, C.POINTER(MlaPool)]),
    "inf_qk_rms_norm_rope": (_I, [_P, _P, _P, _F, _I, C.POINTER(RopeTable), _I, _I, _I, _I, _P]),
    "inf_laguna_qk_rms_norm_rope_pair": (_I, [_P, _P, _P, _P, _P, _F, _I, C.POINTER(RopeTable), _I, _I, _I, _I, _I,
                                              _P, _P]),
    "inf_rope_append_gqa": (_I, [_P, _P, _P, _P, _I, _P, _P, _F, C.POINTER(RopeTable), C.POINTER(KvPool),
                                 C.POINTER(PageTable), _I, _I, _P, _P]),
    "inf_kv_pool_fp8_create": (_I, [_P, _I, _I, _I, _I, _F, _F, C.POINTER(KvPoolFp8)]),
    "inf_kv_pool_fp8_destroy": (_I, [_P, C.POINTER(KvPoolFp8)]),
    "inf_rope_append_gqa_fp8": (_I, [_P, _P, _P, _P, _I, _P, _P, _F, C.POINTER(RopeTable), C.POINTER(KvPoolFp8),
                                     C.POINTER(PageTable), _I, _I, _P, _P, _P]),
    "inf_gqa_decode_paged_fp8": (_I, [_P, _P, _P, _P, C.POINTER(KvPoolFp8), C.POINTER(PageTable), _I, _I, _I, _I, _P, _F,
                                      _P, _I]),
    "inf_rope_slice": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _F]),
    "inf_mla_kv_postprocess_append": (_I, [_P, _P, _P, _F, _F, C.POINTER(MlaPool), C.POINTER(PageTable), _I, _P, _P]),
    "inf_gqa_decode_paged": (_I, [_P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _I, _I, _I, _P, _F, _P, _I]),
    "inf_gqa_decode_paged_peers": (_I, [_P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _I, _I, _I, _P, _F, _P, _I,
                                        _P, _I]),
    "inf_gqa_decode_workspace_bytes": (C.c_size_t, [_I, _I, _I, _I, _I]),
    "inf_gqa_decode_paged_static": (_I, [_P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _I, _I, _I, _P, _F, _P,
                                         _I]),
    "inf_gqa_prefill_paged": (_I, [_P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _I, _I, _P, _F, _P, _I]),
    "inf_laguna_gated_gqa_f16_attention": (_I, [_P, _P, _P, _P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _I,
                                                _I, _I, _P]),
    "inf_mla_decode_absorbed": (_I, [_P, _P, C.POINTER(MlaPool), C.POINTER(PageTable), _I, _I, _I, _F, _P, _I]),
    "inf_mla_decode_absorbed_selected": (_I, [_P, _P, C.POINTER(MlaPool), C.POINTER(PageTable), _P, _P, _I, _I, _F, _P,
                                              _I]),
    "inf_selected_decode_attention": (_I, [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "inf_selected_sequence_attention": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "inf_dsa_scores": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "inf_dsa_topk": (_I, [_P, _P, _I, _I, _I, _P, _I]),
    "inf_dsa_index_key": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _P]),
    "inf_dsa_query_weights": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P]),
    "inf_fp8_e4m3fn_encode": (_I, [_P, _P, _L, _F, _P]),
    "inf_fp8_e4m3fn_decode": (_I, [_P, _P, _L, _F, _P]),
    "inf_kv_pool_from_fp8": (_I, [_P, _P, _P, _F, _F, C.POINTER(KvPool)]),
    "inf_q8_rows_encode": (_I, [_P, _P, _L, _I, _P]),
    "inf_q8_rows_decode": (_I, [_P, _P, _L, _I, _P]),
    "inf_mla_pool_thaw_q8_rows": (_I, [_P, _P, _P, C.POINTER(MlaPool), C.POINTER(PageTable), _I, _I]),
    "inf_q8_0_packed_heads_matvec": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "inf_q8_0_absorbed_mla": (_I, [_P, _P, _P, _P, _P, _P, _P, C.POINTER(MlaPool), C.POINTER(PageTable), _I, _I, _I,
                                   _I, _I, _I, _P]),
    "inf_mla_prefill_causal": (_I, [_P, _P, _L, _L, _P, _L, _L, _P, _L, _P, _L, _L, _I, _I, _I, _I, _I, _F, _P, _L,
                                    _L, _I]),
    "inf_linearize_paged": (_I, [_P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _P]),
    "inf_paged_decode_attention_resident": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "inf_comm_unique_id": (_I, [_P, _P]),
    "inf_comm_init": (_I, [_P, _P, _I, _I, C.POINTER(_P)]),
    "inf_comm_destroy": (_I, [_P]),
    "inf_allgather_heads": (_I, [_P, _P, _P, C.c_size_t]),
    "inf_comm_barrier": (_I, [_P]),
    "inf_comm_barrier_is_p2p": (_I, [_P]),
    "inf_peer_export": (_I, [_P, _P, _P]),
    "inf_peer_open": (_I, [_P, _P, C.POINTER(_P)]),
    "inf_peer_close": (_I, [_P, _P, _P]),
    "inf_mla_prefill_causal_peers": (_I, [_P, _P, _L, _L, _P, _L, _L, _P, _L, _P, _L, _L, _I, _I, _I, _I, _I, _F, _P, _L,
                                          _L, _I, _P, _I]),
    "inf_gqa_prefill_paged_peers": (_I, [_P, _P, C.POINTER(KvPool), C.POINTER(PageTable), _I, _I, _I, _P, _F, _P, _I, _L,
                                         _P, _I]),
    "inf_paged_index_create": (_I, [_I, _I, _I, _I, C.POINTER(_P)]),
    "inf_paged_index_destroy": (_I, [_P]),
    "inf_paged_index_last_error": (C.c_char_p, [_P]),
    "inf_paged_index_append": (_I, [_P, _I, _I, C.POINTER(_I), C.POINTER(_I)]),
    "inf_paged_index_locate": (_I, [_P, _I, _I, C.POINTER(_I), C.POINTER(_I)]),
    "inf_paged_index_len": (_I, [_P, _I]),
    "inf_paged_index_page_count": (_I, [_P, _I]),
    "inf_paged_index_free_pages": (_I, [_P]),
    "inf_paged_index_release": (_I, [_P, _I]),
    "inf_paged_index_trim": (_I, [_P, _I, _I, C.POINTER(_I)]),
    "inf_paged_index_checkpoint": (_I, [_P, _I]),
    "inf_paged_index_restore": (_I, [_P, _I]),
    "inf_paged_index_arrays": (_I, [_P, C.POINTER(_P), C.POINTER(_P), C.POINTER(_I), C.POINTER(_I)]),
}

_lib = None


def load() -> C.CDLL:
    """Load the CUDA library; raise loudly if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m inferno_b200.build` "
                              "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
