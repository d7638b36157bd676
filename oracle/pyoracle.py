"""ctypes binding of the CPU oracle (oracle/liboracle.so) -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg import this
module.  Arrays are numpy; fp16 data travels as numpy float16 viewed as uint16.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile oracle.cpp with the Makefile beside it (no-op when up to date)."""
    src_mtime = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("oracle.cpp", "oracle.h"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_mtime:
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def _p(a, dtype=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    if dtype is not None:
        assert a.dtype == dtype, (a.dtype, dtype)
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def use_all_host_threads() -> int:
    """Make later oracle calls use every core this process may run on, whatever OMP_NUM_THREADS says (torchrun
    exports OMP_NUM_THREADS=1 to its workers).  Returns the thread count now in use."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_threads(C.c_int(n))
    return max_threads()


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    f = lib().orc_f32_to_f16
    return np.array([f(float(v)) for v in x.ravel()], dtype=np.uint16).reshape(x.shape)


def round_f16(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().orc_round_to_f16(_p(x), _p(out), C.c_int64(x.size))
    return out


def fill_normal(shape, seed: int, sigma: float = 1.0, round_to_f16: bool = True) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    lib().orc_fill_normal(_p(out), C.c_int64(out.size), C.c_uint64(seed), C.c_float(sigma), C.c_int(int(round_to_f16)))
    return out


def permutation(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int32)
    lib().orc_permutation(_p(out), C.c_int32(n), C.c_uint64(seed))
    return out


def uniform_int(n: int, lo: int, hi: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.int32)
    lib().orc_uniform_int(_p(out), C.c_int32(n), C.c_int32(lo), C.c_int32(hi), C.c_uint64(seed))
    return out


def default_inv_freq(theta: float, rotary_dim: int) -> np.ndarray:
    out = np.empty(rotary_dim // 2, dtype=np.float32)
    lib().orc_default_inv_freq(C.c_float(theta), C.c_int(rotary_dim), _p(out))
    return out


def yarn_inv_freq(theta, rotary_dim, factor, original_context, beta_fast, beta_slow) -> np.ndarray:
    out = np.empty(rotary_dim // 2, dtype=np.float32)
    lib().orc_yarn_inv_freq(C.c_float(theta), C.c_int(rotary_dim), C.c_float(factor), C.c_float(original_context),
                            C.c_float(beta_fast), C.c_float(beta_slow), _p(out))
    return out


def qk_norm_rope(x, norm_weight, inv_freq, rotary_dim, position_offset, eps=1e-6, factor=1.0, positions=None):
    """x [B,T,H,D] -> same shape.  positions (int32 [B]) overrides position_offset per batch row."""
    x = _f32(x)
    B, T, H, D = x.shape
    out = np.empty_like(x)
    w = _f32(norm_weight)
    inv_freq = _f32(inv_freq)
    if positions is None:
        lib().orc_qk_norm_rope_half_split(_p(x), _p(w), _p(inv_freq), _p(out), C.c_int64(B * T * H), C.c_int(T),
                                          C.c_int(H), C.c_int(D), C.c_int(rotary_dim), C.c_int(position_offset),
                                          C.c_float(eps), C.c_float(factor))
    else:
        pos = _i32(positions)
        lib().orc_qk_norm_rope_half_split_pos(_p(x), _p(w), _p(inv_freq), _p(out), C.c_int(B), C.c_int(T), C.c_int(H),
                                              C.c_int(D), C.c_int(rotary_dim), _p(pos), C.c_float(eps),
                                              C.c_float(factor))
    return out


def rope_slice_glm(x, position_offset, theta):
    x = _f32(x)
    B, T, H, R = x.shape
    out = np.empty_like(x)
    lib().orc_rope_slice_glm(_p(x), _p(out), C.c_int(B), C.c_int(T), C.c_int(H), C.c_int(R), C.c_int(position_offset),
                             C.c_float(theta))
    return out


def mla_kv_postprocess(x, norm_weight, tokens, latent_dim, rope_dim, position_offset, theta, eps):
    x = _f32(x)
    rows = x.size // (latent_dim + rope_dim)
    lat = np.empty((rows, latent_dim), dtype=np.float32)
    rope = np.empty((rows, rope_dim), dtype=np.float32)
    w = _f32(norm_weight)
    lib().orc_mla_kv_postprocess(_p(x), _p(w), _p(lat), _p(rope), C.c_int64(rows), C.c_int(tokens),
                                 C.c_int(latent_dim), C.c_int(rope_dim), C.c_int(position_offset), C.c_float(theta),
                                 C.c_float(eps))
    return lat, rope


def gqa_ring_attention(q, k, v, gate, cached_k, cached_v, past_tokens, stored_tokens, capacity, sliding_window=0,
                       fuse_append=True):
    """q [B,T,Hq,D]; k,v [B,T,Hkv,D]; cached_* uint16 [B,capacity,Hkv,D] (modified in place)."""
    q, k, v, gate = _f32(q), _f32(k), _f32(v), _f32(gate)
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    out = np.empty_like(q)
    lib().orc_gqa_ring_attention(_p(q), _p(k), _p(v), _p(gate), _p(cached_k, np.uint16), _p(cached_v, np.uint16),
                                 _p(out), C.c_int(B), C.c_int(Hq), C.c_int(Hkv), C.c_int(D), C.c_int(T),
                                 C.c_int(past_tokens), C.c_int(stored_tokens), C.c_int(capacity),
                                 C.c_int(sliding_window), C.c_int(int(fuse_append)))
    return out


def test_cpu_gqa(q, k, v, gate, q_heads, kv_heads, head_dim, sliding_window=0, last_only=False):
    q, k, v, gate = _f32(q), _f32(k), _f32(v), _f32(gate)
    tokens = k.size // (kv_heads * head_dim)
    out = np.empty((q_heads, head_dim) if last_only else (tokens, q_heads, head_dim), dtype=np.float32)
    lib().orc_test_cpu_gqa(_p(q), _p(k), _p(v), _p(gate), _p(out), C.c_int(tokens), C.c_int(q_heads),
                           C.c_int(kv_heads), C.c_int(head_dim), C.c_int(sliding_window), C.c_int(int(last_only)))
    return out


def gqa_ring_decode_segmented(q, k, v, gate, cached_k, cached_v, past_tokens, cached_start, cached_count, capacity,
                              segment_tokens):
    q, k, v, gate = _f32(q), _f32(k), _f32(v), _f32(gate)
    B, Hq, D = q.shape[0], q.shape[-2], q.shape[-1]
    Hkv = k.shape[-2]
    out = np.empty((B, Hq, D), dtype=np.float32)
    lib().orc_gqa_ring_decode_segmented(_p(q), _p(k), _p(v), _p(gate), _p(cached_k, np.uint16),
                                        _p(cached_v, np.uint16), _p(out), C.c_int(B), C.c_int(Hq), C.c_int(Hkv),
                                        C.c_int(D), C.c_int(past_tokens), C.c_int(cached_start),
                                        C.c_int(cached_count), C.c_int(capacity), C.c_int(segment_tokens))
    return out


def gqa_paged_attention(q, k, v, gate, k_pool, v_pool, page_table, past_tokens, page_size, sliding_window=0,
                        fuse_append=True, scale=0.0, threads=0):
    """q [B,T,Hq,D]; k,v [B,T,Hkv,D] f32; pools uint16 [pages,Hkv,P,D] (modified in place when appending)."""
    q, k, v, gate = _f32(q), _f32(k), _f32(v), _f32(gate)
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    pt = _i32(page_table)
    past = _i32(past_tokens)
    out = np.empty_like(q)
    lib().orc_gqa_paged_attention(_p(q), _p(k), _p(v), _p(gate), _p(k_pool, np.uint16), _p(v_pool, np.uint16), _p(pt),
                                  C.c_int(pt.shape[1]), _p(past), _p(out), C.c_int(B), C.c_int(Hq), C.c_int(Hkv),
                                  C.c_int(D), C.c_int(page_size), C.c_int(T), C.c_int(sliding_window),
                                  C.c_int(int(fuse_append)), C.c_float(scale), C.c_int(threads))
    return out


def linearize_paged(pool, page_table, tokens, page_size):
    pt = _i32(page_table)
    B = pt.shape[0]
    _, Hkv, P, D = pool.shape
    out = np.empty((B, Hkv, tokens, D), dtype=np.uint16)
    lib().orc_linearize_paged(_p(pool, np.uint16), _p(pt), C.c_int(pt.shape[1]), _p(out), C.c_int(B), C.c_int(Hkv),
                              C.c_int(tokens), C.c_int(page_size), C.c_int(D))
    return out


def paged_decode_mha_f16(q, paged_k, cur_k, paged_v, cur_v, past_tokens, page_size):
    q, cur_k, cur_v = _f32(q), _f32(cur_k), _f32(cur_v)
    B, H, D = q.shape
    Dv = cur_v.shape[-1]
    out = np.empty((B, H, Dv), dtype=np.float32)
    lib().orc_paged_decode_mha_f16(_p(q), _p(paged_k, np.uint16), _p(cur_k), _p(paged_v, np.uint16), _p(cur_v),
                                   _p(out), C.c_int(B), C.c_int(H), C.c_int(past_tokens), C.c_int(page_size),
                                   C.c_int(D), C.c_int(Dv))
    return out


def q8_0_heads_matvec(weights: np.ndarray, x, heads, in_features, out_features):
    x = _f32(x)
    rows = x.size // (heads * in_features)
    out = np.empty((rows, heads, out_features), dtype=np.float32)
    w = np.ascontiguousarray(weights, dtype=np.uint8)
    lib().orc_q8_0_heads_matvec(_p(w), _p(x), _p(out), C.c_int64(rows), C.c_int(heads), C.c_int(in_features),
                                C.c_int(out_features))
    return out


def mla_absorbed_f32(q_latent, q_rope, paged_latent, cur_latent, paged_rope, cur_rope, batch, heads, q_tokens,
                     past_tokens, page_size, latent_dim, rope_dim, scale_dim):
    a = [_f32(t) for t in (q_latent, q_rope, paged_latent, cur_latent, paged_rope, cur_rope)]
    out = np.empty((batch, q_tokens, heads, latent_dim), dtype=np.float32)
    lib().orc_mla_absorbed_f32(_p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(a[5]), _p(out), C.c_int(batch),
                               C.c_int(heads), C.c_int(q_tokens), C.c_int(past_tokens), C.c_int(page_size),
                               C.c_int(latent_dim), C.c_int(rope_dim), C.c_int(scale_dim))
    return out


def mla_absorbed_paged(q, cur_rows, pool, page_table, past_tokens, page_size, latent_dim, rope_dim, scale,
                       fuse_append=True, threads=0):
    """q [B,T,H,L+R] f32; cur_rows [B,T,L+R] f32; pool uint16 [pages,P,L+R]."""
    q, cur_rows = _f32(q), _f32(cur_rows)
    B, T, H, _ = q.shape
    pt = _i32(page_table)
    past = _i32(past_tokens)
    out = np.empty((B, T, H, latent_dim), dtype=np.float32)
    lib().orc_mla_absorbed_paged(_p(q), _p(cur_rows), _p(pool, np.uint16), _p(pt), C.c_int(pt.shape[1]), _p(past),
                                 _p(out), C.c_int(B), C.c_int(H), C.c_int(T), C.c_int(page_size), C.c_int(latent_dim),
                                 C.c_int(rope_dim), C.c_float(scale), C.c_int(int(fuse_append)), C.c_int(threads))
    return out


def causal_mha(q, k_nope, k_rope, v, scale, rows=None, threads=0):
    """q [T,H,dn+dr]; k_nope [T,H,dn]; k_rope [T,dr] or None; v [T,H,dv]; rows int32 list or None."""
    q, k_nope, v = _f32(q), _f32(k_nope), _f32(v)
    T, H, dqk = q.shape
    dn = k_nope.shape[2]
    dr = dqk - dn
    kr = _f32(k_rope) if dr else None
    dv = v.shape[2]
    r = _i32(rows) if rows is not None else None
    n = len(r) if r is not None else T
    out = np.empty((n, H, dv), dtype=np.float32)
    lib().orc_causal_mha(_p(q), _p(k_nope), _p(kr), _p(v), _p(out), C.c_int(T), C.c_int(H), C.c_int(dn), C.c_int(dr),
                         C.c_int(dv), C.c_float(scale), _p(r), C.c_int(n), C.c_int(threads))
    return out


def dsa_scores(q, weights, past_keys, current_key):
    """dsa_scores_f32_kernel (crates/backend/src/metal/kernels/dsa_kernels.metal:137-176), numpy restatement:
    q [B,H,D], weights [B,H], past_keys [B,past,D], current_key [B,D] -> [B, past+1] f32, accumulating in the
    kernel's order (dims, then heads) in f32."""
    q, weights, current_key = _f32(q), _f32(weights), _f32(current_key)
    keys = np.concatenate([_f32(past_keys), current_key[:, None, :]], axis=1)
    scale = np.float32(1.0) / np.sqrt(np.float32(q.shape[2]))
    dots = np.einsum("bhd,btd->bth", q, keys, dtype=np.float32) * scale
    return np.einsum("bth,bh->bt", np.maximum(dots, np.float32(0.0)), weights, dtype=np.float32).astype(np.float32)


def dsa_topk(scores, top_k):
    """Top-k ids best first under dsa_precedes (dsa_kernels.metal:182-196): higher score first, ties by lower id;
    missing entries 0xffffffff.  uint32 [B, top_k]."""
    scores = _f32(scores)
    B, n = scores.shape
    out = np.full((B, top_k), 0xFFFFFFFF, np.uint32)
    ids = np.arange(n)
    for b in range(B):
        order = np.lexsort((ids, -scores[b].astype(np.float64)))[:top_k]
        out[b, :len(order)] = order.astype(np.uint32)
    return out


def q8_rows_encode(x):
    """encode_q8_rows (crates/cache/src/cold_kv.rs:1624-1655): f32 [rows, dim] -> uint8 [rows, 4 + dim];
    scale = max|x| / 127 (1.0 for a zero row), value = round-half-away(x / scale) clamped to +-127, all in f32."""
    x = _f32(x)
    rows, dim = x.shape
    m = np.abs(x).max(axis=1).astype(np.float32)
    scale = np.where(m == 0, np.float32(1.0), (m / np.float32(127.0)).astype(np.float32)).astype(np.float32)
    r = (x / scale[:, None]).astype(np.float32)
    qv = np.clip(np.sign(r) * np.floor(np.abs(r) + np.float32(0.5)), -127, 127).astype(np.int8)
    out = np.empty((rows, dim + 4), np.uint8)
    out[:, :4] = scale.astype("<f4").view(np.uint8).reshape(rows, 4)
    out[:, 4:] = qv.view(np.uint8)
    return out


def q8_rows_decode(payload, dim):
    """decode_q8_rows (cold_kv.rs:1657-1703) / q8_rows_to_f32_kernel (cast_kernels.metal:31-56)."""
    p = np.ascontiguousarray(payload, dtype=np.uint8).reshape(-1, dim + 4)
    scale = p[:, :4].copy().view("<f4").reshape(-1).astype(np.float32)
    return (p[:, 4:].view(np.int8).astype(np.float32) * scale[:, None]).astype(np.float32)


def selected_attention(q, sel_k, sel_v, cur_k, cur_v, include_current=True):
    """kernels/attention_kernels.metal:605-721 / :723-968: q [B,H,T,D], sel_k [B,H,S,D], sel_v [B,H,S,Dv] (or None for
    S = 0), cur_k [B,H,T,D], cur_v [B,H,T,Dv] -> [B,H,T,Dv]."""
    q, cur_k, cur_v = _f32(q), _f32(cur_k), _f32(cur_v)
    B, H, T, D = q.shape
    Dv = cur_v.shape[3]
    S = 0 if sel_k is None else sel_k.shape[2]
    sel_k, sel_v = _f32(sel_k), _f32(sel_v)
    out = np.empty((B, H, T, Dv), np.float32)
    lib().orc_selected_attention_f32(_p(q), _p(sel_k), _p(sel_v), _p(cur_k), _p(cur_v), _p(out), C.c_int(B), C.c_int(H),
                                     C.c_int(S), C.c_int(T), C.c_int(D), C.c_int(Dv), C.c_int(int(include_current)))
    return out


def gqa_paged_attention_fp8(q, k, v, gate, k_pool, v_pool, key_scale, value_scale, page_table, past_tokens, page_size,
                            sliding_window=0, fuse_append=True, scale=0.0, threads=0):
    """laguna_gated_gqa_fp8_attention (fp8_attention_kernels.metal:70-263) over pages: q [B,T,Hq,D]; k, v [B,T,Hkv,D]
    f32; pools uint8 [pages,Hkv,P,D] (modified in place when appending)."""
    q, k, v, gate = _f32(q), _f32(k), _f32(v), _f32(gate)
    B, T, Hq, D = q.shape
    Hkv = k.shape[2]
    pt = _i32(page_table)
    past = _i32(past_tokens)
    out = np.empty_like(q)
    lib().orc_gqa_paged_attention_fp8(_p(q), _p(k), _p(v), _p(gate), _p(k_pool, np.uint8), _p(v_pool, np.uint8),
                                      C.c_float(key_scale), C.c_float(value_scale), _p(pt), C.c_int(pt.shape[1]),
                                      _p(past), _p(out), C.c_int(B), C.c_int(Hq), C.c_int(Hkv), C.c_int(D),
                                      C.c_int(page_size), C.c_int(T), C.c_int(sliding_window),
                                      C.c_int(int(fuse_append)), C.c_float(scale), C.c_int(threads))
    return out


def fp8_codec_c(values=None, bits=None):
    """The C restatement of the codec, element by element (pins it against the numpy statement below)."""
    L = lib()
    L.orc_fp8_e4m3fn_decode.restype = C.c_float
    L.orc_fp8_e4m3fn_decode.argtypes = [C.c_uint8]
    L.orc_fp8_e4m3fn_encode.restype = C.c_uint8
    L.orc_fp8_e4m3fn_encode.argtypes = [C.c_float]
    if bits is not None:
        return np.array([L.orc_fp8_e4m3fn_decode(int(b)) for b in np.asarray(bits).ravel()], np.float32)
    return np.array([L.orc_fp8_e4m3fn_encode(float(x)) for x in np.asarray(values, np.float32).ravel()], np.uint8)


def fp8_e4m3fn_decode(bits):
    """laguna_fp8_e4m3fn_decode (crates/backend/src/metal/kernels/fp8_attention_kernels.metal:11-27): uint8 -> f32."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.int32)
    sign, exponent, mant = b >> 7, (b >> 3) & 15, b & 7
    mag = np.where(exponent == 0, mant * np.float32(2.0 ** -9),
                   (1.0 + mant * 0.125) * np.exp2((exponent - 7).astype(np.float64))).astype(np.float32)
    out = np.where(sign == 1, -mag, mag).astype(np.float32)
    return np.where((exponent == 15) & (mant == 7), np.float32(0.0), out).astype(np.float32)  # both NaN codes read +0


def fp8_e4m3fn_encode(x):
    """laguna_fp8_e4m3fn_encode (fp8_attention_kernels.metal:29-54): f32 -> uint8 (the caller divides by the scale)."""
    x = _f32(x)
    out = np.zeros(x.shape, np.uint8)
    ok = ~(np.isnan(x) | (x == 0))
    sign = np.where(x < 0, 0x80, 0).astype(np.uint32)
    mag = np.minimum(np.abs(x), np.float32(448.0)).astype(np.float32)
    small = mag < np.float32(0.015625)
    m_small = np.minimum(np.rint(mag.astype(np.float64) * 512.0), 8).astype(np.uint32)
    with np.errstate(divide="ignore", invalid="ignore"):
        _, e2 = np.frexp(np.where(ok, mag, np.float32(1.0)).astype(np.float64))  # mag = m * 2^e2, m in [0.5, 1)
    e = e2 - 1
    norm = np.where(ok, mag, np.float32(1.0)).astype(np.float64) * np.exp2(-e.astype(np.float64))
    mant = np.rint((norm - 1.0) * 8.0).astype(np.int64)
    exponent = (e + 7).astype(np.int64)
    bump = mant == 8
    mant = np.where(bump, 0, mant)
    exponent = np.where(bump, exponent + 1, exponent)
    sat = (exponent > 15) | ((exponent == 15) & (mant > 6))
    exponent = np.where(sat, 15, exponent)
    mant = np.where(sat, 6, mant)
    normal = (sign | (exponent.astype(np.uint32) << 3) | mant.astype(np.uint32)).astype(np.uint32)
    res = np.where(small, sign | m_small, normal)
    out[ok] = res[ok].astype(np.uint8)
    return out


def _libm_powf(x, y):
    import ctypes
    import ctypes.util
    libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
    libm.powf.restype = ctypes.c_float
    libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
    return libm.powf(x, y)


def dsa_rotate_interleaved(values, rope_dim, position, theta):
    """rotate_interleaved_pair_range (crates/model/src/indexer.rs:483-514): pairs (2p, 2p+1) of the first rope_dim
    values rotated by position * theta^(-2p/rope_dim), written as halves (p, rope_dim/2 + p); f32 arithmetic."""
    out = _f32(values).copy()
    pairs = rope_dim // 2
    p = np.arange(pairs)
    # f32::powf in the reference is libm's powf; numpy's float32 power may differ from it in the last bit, which at
    # position 1000 is already 6e-5 rad of angle, so the frequencies come from libm itself
    freq = np.array([np.float32(1.0) / np.float32(_libm_powf(float(np.float32(theta)), float(np.float32(2 * k) / np.float32(rope_dim))))
                     for k in p], dtype=np.float32)
    angle = (np.float32(position) * freq).astype(np.float32)
    c, s = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    x0, x1 = out[..., 0:rope_dim:2].copy(), out[..., 1:rope_dim:2].copy()
    out[..., :pairs] = x0 * c - x1 * s
    out[..., pairs:rope_dim] = x1 * c + x0 * s
    return out


def dsa_index_key(raw_key, weight, bias, rope_dim, position_offset, theta, eps=1e-6):
    """DsaIndexer::key_f32 after the projection (indexer.rs:190-203): layer_norm_last_dim (:397-428) then
    apply_interleaved_rope_to_key (:458-481).  raw_key [B,T,D] -> f32 [B,T,D]."""
    x = _f32(raw_key)
    mean = (x.sum(axis=-1, dtype=np.float32) / np.float32(x.shape[-1]))[..., None]
    var = (np.square(x - mean).sum(axis=-1, dtype=np.float32) / np.float32(x.shape[-1]))[..., None]
    inv_std = np.float32(1.0) / np.sqrt(var + np.float32(eps))
    y = ((x - mean) * inv_std * _f32(weight) + _f32(bias)).astype(np.float32)
    out = np.empty_like(y)
    for t in range(y.shape[1]):
        out[:, t] = dsa_rotate_interleaved(y[:, t], rope_dim, position_offset + t, theta)
    return out


def dsa_query_weights(hidden_states, q_raw, weights_proj, heads, head_dim, rope_dim, position_offset, theta):
    """indexer_weights (indexer.rs:516-543) and apply_interleaved_rope_to_query (:430-456): hidden_states [B,hidden],
    q_raw [B,heads*head_dim], weights_proj [hidden,heads] -> (q [B,heads,head_dim], weights [B,heads])."""
    h, proj = _f32(hidden_states), _f32(weights_proj)
    scale = np.float32(1.0) / np.sqrt(np.float32(heads))
    w = ((h.astype(np.float64) @ proj.astype(np.float64)).astype(np.float32) * scale).astype(np.float32)
    q = _f32(q_raw).reshape(h.shape[0], heads, head_dim)
    return dsa_rotate_interleaved(q, rope_dim, position_offset, theta), w


def dsa_decode_topk(hidden_states, q_raw, past_keys, current_key, weights_proj, heads, head_dim, rope_dim,
                    position_offset, theta, top_k):
    """Backend::dsa_decode_topk_device (crates/backend/src/backend.rs:2074) as one chain on the CPU."""
    B = np.asarray(hidden_states).shape[0]
    q, w = dsa_query_weights(np.reshape(hidden_states, (B, -1)), np.reshape(q_raw, (B, -1)), weights_proj, heads,
                             head_dim, rope_dim, position_offset, theta)
    return dsa_topk(dsa_scores(q, w, past_keys, np.reshape(current_key, (B, head_dim))), top_k)

