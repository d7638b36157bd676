"""Pins the CPU oracle to the reference's own known-answer tests.

Every case below restates one test of the reference from its closed-form inputs (index
ramps and modular patterns, so nothing is copied but the formulas) and checks the oracle
with the tolerance that test uses.  The independent statements the reference writes
inside its test modules (two-pass softmax in f32) are re-derived here in numpy, so the
oracle is checked against them and against its own C restatement of them.
"""
import math

import numpy as np
import pytest

from oracle import pyoracle as orc

HEAD_DIM = 128
KV_HEADS = 8
SLIDING_WINDOW = 512  # crates/backend/src/metal/f16_attention.rs:30


def patterned(n, period, center, divisor):
    # metal/f16_attention.rs:1135-1139
    idx = np.arange(n)
    return ((idx % period).astype(np.float32) - np.float32(center)) / np.float32(divisor)


def np_gqa_row(q, k, v, gate, token, q_heads, first_key=0):
    """numpy two-pass statement of one token row (metal/f16_attention.rs:1079-1133)."""
    hpk = q_heads // KV_HEADS
    out = np.zeros((q_heads, HEAD_DIM), np.float32)
    scale = np.float32(1.0 / math.sqrt(HEAD_DIM))
    for h in range(q_heads):
        kv = h // hpk
        qv = q[token, h]
        keys = k[first_key:token + 1, kv]
        scores = (keys @ qv).astype(np.float32) * scale
        w = np.exp(scores - scores.max()).astype(np.float32)
        gain = np.float32(math.log1p(math.exp(float(gate[token, h]))))
        out[h] = (w @ v[first_key:token + 1, kv]) / w.sum() * gain
    return out


# ------------------------------------------------------------------ fp16
def test_f16_conversion_matches_ieee_rne():
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 100,
        rng.standard_normal(20000).astype(np.float32) * 1e-6,
        np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 1e9, -1e9, 5.9604645e-8, 2.9802322e-8, 2.98023224e-8 * 1.0001,
                  6.1035156e-5, 6.0975552e-5, 1.0009766, 1.00048828125, 1.00146484375, np.inf, -np.inf], np.float32),
    ])
    got = orc.round_f16(vals)
    want = vals.astype(np.float16).astype(np.float32)
    assert np.array_equal(got, want)
    bits = orc.f32_to_f16_bits(vals[:500])
    assert np.array_equal(bits, vals[:500].astype(np.float16).view(np.uint16))


# ------------------------------------------------------------------ Laguna GQA
def test_ln2_identities_f16_cache_preserves_prefill_values():
    # metal/f16_attention.rs:708-767
    Hq = 48
    ck = np.zeros((1, 4, KV_HEADS, HEAD_DIM), np.uint16)
    cv = np.zeros_like(ck)
    q = np.zeros((1, 2, Hq, HEAD_DIM), np.float32)
    k = np.zeros((1, 2, KV_HEADS, HEAD_DIM), np.float32)
    v = np.ones((1, 2, KV_HEADS, HEAD_DIM), np.float32)
    v[0, 1] = 3.0
    gate = np.zeros((1, 2, Hq), np.float32)
    out = orc.gqa_ring_attention(q, k, v, gate, ck, cv, 0, 0, 4)
    ln2 = math.log(2.0)
    assert abs(out[0, 0, 0, 0] - ln2) <= 1e-4
    assert abs(out[0, 1, 0, 0] - 2 * ln2) <= 1e-4
    out = orc.gqa_ring_attention(np.zeros((1, 1, Hq, HEAD_DIM)), np.zeros((1, 1, KV_HEADS, HEAD_DIM)),
                                 np.full((1, 1, KV_HEADS, HEAD_DIM), 5.0), np.zeros((1, 1, Hq)), ck, cv, 2, 2, 4)
    assert abs(out[0, 0, 0, 0] - 3 * ln2) <= 1e-4


def test_prefill_matches_nonuniform_cpu_reference():
    # metal/f16_attention.rs:792-842, tolerance max(5e-4, 5e-4*|x|)
    T, Hq = 8, 48
    q = patterned(T * Hq * HEAD_DIM, 17, 8, 16.0).reshape(1, T, Hq, HEAD_DIM)
    k = patterned(T * KV_HEADS * HEAD_DIM, 13, 6, 16.0).reshape(1, T, KV_HEADS, HEAD_DIM)
    v = patterned(T * KV_HEADS * HEAD_DIM, 11, 5, 8.0).reshape(1, T, KV_HEADS, HEAD_DIM)
    gate = patterned(T * Hq, 7, 3, 10.0).reshape(1, T, Hq)
    ck = np.zeros((1, T, KV_HEADS, HEAD_DIM), np.uint16)
    cv = np.zeros_like(ck)
    got = orc.gqa_ring_attention(q, k, v, gate, ck, cv, 0, 0, T)
    want_c = orc.test_cpu_gqa(q, k, v, gate, Hq, KV_HEADS, HEAD_DIM)
    want_np = np.stack([np_gqa_row(q[0], k[0], v[0], gate[0], t, Hq) for t in range(T)])
    for want in (want_c, want_np):
        tol = np.maximum(5e-4, np.abs(want) * 5e-4)
        assert np.all(np.abs(got[0] - want) <= tol)
    # the fused append stored RNE fp16 of the current rows
    assert np.array_equal(ck.view(np.float16), k.astype(np.float16))


@pytest.mark.parametrize("sliding,q_heads,tokens,segmented", [
    (False, 48, 37, False), (False, 48, 37, True), (True, 64, 600, True), (True, 72, 600, False)])
def test_decode_step_matches_nonuniform_cpu_reference(sliding, q_heads, tokens, segmented):
    # metal/f16_attention.rs:955-1075, tolerance max(2e-3, 2e-3*|x|)
    q = patterned(tokens * q_heads * HEAD_DIM, 17, 8, 16.0).reshape(1, tokens, q_heads, HEAD_DIM)
    k = patterned(tokens * KV_HEADS * HEAD_DIM, 13, 6, 16.0).reshape(1, tokens, KV_HEADS, HEAD_DIM)
    v = patterned(tokens * KV_HEADS * HEAD_DIM, 11, 5, 8.0).reshape(1, tokens, KV_HEADS, HEAD_DIM)
    gate = patterned(tokens * q_heads, 7, 3, 10.0).reshape(1, tokens, q_heads)
    window = SLIDING_WINDOW if sliding else 0
    capacity = SLIDING_WINDOW if sliding else tokens
    ck = np.zeros((1, capacity, KV_HEADS, HEAD_DIM), np.uint16)
    cv = np.zeros_like(ck)
    prefill = tokens - 1
    orc.gqa_ring_attention(q[:, :prefill], k[:, :prefill], v[:, :prefill], gate[:, :prefill], ck, cv, 0, 0, capacity,
                           window)
    stored = min(prefill, capacity)
    if segmented:
        cached_count = prefill if not sliding else min(prefill, capacity - 1)  # metal/f16_attention.rs:459-464
        got = orc.gqa_ring_decode_segmented(q[:, prefill:], k[:, prefill:], v[:, prefill:], gate[:, prefill:], ck, cv,
                                            prefill, prefill - cached_count, cached_count, capacity, 16)[0]
    else:
        got = orc.gqa_ring_attention(q[:, prefill:], k[:, prefill:], v[:, prefill:], gate[:, prefill:], ck, cv,
                                     prefill, stored, capacity, window)[0, 0]
    want_c = orc.test_cpu_gqa(q, k, v, gate, q_heads, KV_HEADS, HEAD_DIM, window, last_only=True)
    first = 0 if (window == 0 or tokens - 1 < window) else tokens - window
    want_np = np_gqa_row(q[0], k[0], v[0], gate[0], tokens - 1, q_heads, first)
    for want in (want_c, want_np):
        tol = np.maximum(2e-3, np.abs(want) * 2e-3)
        assert np.all(np.abs(got - want) <= tol)


# ------------------------------------------------------------------ RoPE
def np_qk_norm_rope(x, w, pos_off, eps, inv_freq, rotary, factor):
    # metal/rope.rs:828-875 in numpy f32
    B, T, H, D = x.shape
    out = np.zeros_like(x)
    half = rotary // 2
    for b in range(B):
        for t in range(T):
            for h in range(H):
                row = x[b, t, h]
                inv_rms = np.float32(1.0) / np.sqrt(np.float32((row * row).sum(dtype=np.float32) / np.float32(D) + np.float32(eps)))
                n = row * w * inv_rms
                o = n.copy()
                for d in range(rotary):
                    pd = d + half if d < half else d - half
                    rot = -n[pd] if d < half else n[pd]
                    ang = np.float32(pos_off + t) * inv_freq[d % half]
                    o[d] = np.float32(factor) * (n[d] * np.cos(ang, dtype=np.float32) + rot * np.sin(ang, dtype=np.float32))
                out[b, t, h] = o
    return out


@pytest.mark.parametrize("rotary,theta,factor", [(64, 500000.0, 1.3465736), (128, 10000.0, 1.0)])
def test_qk_norm_rope_matches_global_and_sliding_references(rotary, theta, factor):
    # metal/rope.rs:560-619, tolerance 3e-5
    B, T, H, D, pos = 1, 2, 3, 128, 11
    x = ((np.arange(B * T * H * D) % 97).astype(np.float32) - 48.0) / np.float32(31.0)
    x = x.reshape(B, T, H, D)
    w = np.float32(0.75) + (np.arange(D) % 13).astype(np.float32) / np.float32(40.0)
    inv = (1.0 / np.power(np.float32(theta), (2 * np.arange(rotary // 2)).astype(np.float32) / np.float32(rotary))).astype(np.float32)
    assert np.allclose(inv, orc.default_inv_freq(theta, rotary), rtol=1e-6)
    got = orc.qk_norm_rope(x, w, inv, rotary, pos, 1e-6, factor)
    want = np_qk_norm_rope(x, w, pos, 1e-6, inv, rotary, factor)
    assert np.max(np.abs(got - want)) <= 3e-5


def test_qk_pair_shapes():
    # metal/rope.rs:621-710: the pair kernel is the single kernel applied to Q and K rows separately
    D, rotary, theta, factor, pos = 128, 64, 500000.0, 1.3465736, 7
    qv = (((np.arange(2 * 3 * D) % 43).astype(np.float32) - 21.0) / 16.0).reshape(1, 2, 3, D)
    kv = (((np.arange(2 * 8 * D) % 59).astype(np.float32) - 29.0) / 24.0).reshape(1, 2, 8, D)
    qw = np.float32(0.75) + (np.arange(D) % 5).astype(np.float32) * np.float32(0.0625)
    kw = np.float32(0.875) + (np.arange(D) % 7).astype(np.float32) * np.float32(0.03125)
    inv = orc.default_inv_freq(theta, rotary)
    assert np.max(np.abs(orc.qk_norm_rope(qv, qw, inv, rotary, pos, 1e-6, factor) - np_qk_norm_rope(qv, qw, pos, 1e-6, inv, rotary, factor))) <= 3e-5
    assert np.max(np.abs(orc.qk_norm_rope(kv, kw, inv, rotary, pos, 1e-6, factor) - np_qk_norm_rope(kv, kw, pos, 1e-6, inv, rotary, factor))) <= 3e-5


def test_rope_slice_rotates_adjacent_glm_pairs():
    # backend.rs:11285-11303, tolerance 1e-6
    out = orc.rope_slice_glm(np.array([1.0, 2.0, 3.0, 4.0], np.float32).reshape(1, 1, 1, 4), 1, 10000.0).ravel()
    slow = 1.0 / math.sqrt(10000.0)
    want = [math.cos(1.0) - 2 * math.sin(1.0), 2 * math.cos(1.0) + math.sin(1.0),
            3 * math.cos(slow) - 4 * math.sin(slow), 4 * math.cos(slow) + 3 * math.sin(slow)]
    assert np.max(np.abs(out - np.array(want, np.float32))) < 1e-6


def np_rope_slice(x, pos_off, theta):
    # metal/rope.rs:877-912
    B, T, H, R = x.shape
    pc = R // 2
    p = np.arange(pc, dtype=np.float32)
    inv = (np.float32(1.0) / np.power(np.float32(theta), p / np.float32(pc))).astype(np.float32)
    pos = (pos_off + np.arange(T)).astype(np.float32)
    ang = pos[:, None] * inv[None, :]
    c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    e, o = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = e * c[None, :, None, :] - o * s[None, :, None, :]
    out[..., 1::2] = e * s[None, :, None, :] + o * c[None, :, None, :]
    return out


@pytest.mark.parametrize("T,H,R,pos", [(2, 2, 4, 3), (32, 64, 64, 7)])
def test_rope_slice_matches_cpu_reference(T, H, R, pos):
    # metal/rope.rs:720-804, tolerance 1e-5
    n = T * H * R
    x = ((np.arange(n) + 1) / 10.0 if R == 4 else ((np.arange(n) % 251) - 125.0) / 64.0).astype(np.float32)
    x = x.reshape(1, T, H, R)
    assert np.max(np.abs(orc.rope_slice_glm(x, pos, 10000.0) - np_rope_slice(x, pos, 10000.0))) <= 1e-5


def test_yarn_frequencies_contract():
    # crates/config/src/laguna.rs:873-897
    g = orc.yarn_inv_freq(500000.0, 64, 32.0, 8192.0, 32.0, 1.0)
    s = orc.default_inv_freq(10000.0, 128)
    assert len(g) == 32 and len(s) == 64
    assert g[0] == 1.0 and s[0] == 1.0
    assert g[20] != s[20]
    assert np.all(g[:-1] >= g[1:]) and np.all(s[:-1] > s[1:])


def test_mla_kv_postprocess_matches_separate_norm_and_rope():
    # kernels/norm_kernels.metal:52-115 = RMSNorm (:1-50) on the latent + rope_slice on the tail
    rows, T, L, R, pos, theta, eps = 6, 3, 512, 64, 5, 1.0e7, 1e-6
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, L + R)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(L)).astype(np.float32)
    lat, rope = orc.mla_kv_postprocess(x, w, T, L, R, pos, theta, eps)
    lat_np = x[:, :L] * (1.0 / np.sqrt((x[:, :L] ** 2).mean(axis=1, dtype=np.float32) + np.float32(eps)))[:, None] * w
    assert np.max(np.abs(lat - lat_np)) <= 1e-5
    tail = x[:, L:].reshape(rows // T, T, 1, R)
    assert np.max(np.abs(rope.reshape(tail.shape) - orc.rope_slice_glm(tail, pos, theta))) <= 1e-6


# ------------------------------------------------------------------ GLM paged decode, causal softmax
def test_causal_softmax_masks_future_keys():
    # backend.rs:11241-11263: uniform scores -> rows (1), (.5,.5), (1/3,1/3,1/3)
    T = 3
    q = np.zeros((T, 1, 4), np.float32)
    k = np.zeros((T, 1, 4), np.float32)
    v = np.eye(T, dtype=np.float32).reshape(T, 1, T)
    p = orc.causal_mha(q, k, None, v, 0.5)[:, 0, :]
    want = np.array([[1, 0, 0], [.5, .5, 0], [1 / 3, 1 / 3, 1 / 3]], np.float32)
    assert np.max(np.abs(p - want)) < 1e-6


def test_paged_f16_decode_matches_contiguous_on_f16_rounded_past():
    # metal/attention.rs:2742-2859: resident F16 paged decode == dense attention on f16-rounded past K/V, tol 1e-5
    B, H, D, Dv, P, past = 1, 4, 32, 32, 8, 21
    rng = np.random.default_rng(5)
    kp = rng.standard_normal((past, B, H, D)).astype(np.float32) * 0.5
    vp = rng.standard_normal((past, B, H, Dv)).astype(np.float32) * 0.5
    pages = (past + P - 1) // P
    pk = np.zeros((pages, B, H, P, D), np.float16)
    pv = np.zeros((pages, B, H, P, Dv), np.float16)
    for t in range(past):
        pk[t // P, :, :, t % P] = kp[t]
        pv[t // P, :, :, t % P] = vp[t]
    q = rng.standard_normal((B, H, D)).astype(np.float32)
    ck = rng.standard_normal((B, H, D)).astype(np.float32)
    cvv = rng.standard_normal((B, H, Dv)).astype(np.float32)
    got = orc.paged_decode_mha_f16(q, pk.view(np.uint16), ck, pv.view(np.uint16), cvv, past, P)
    kf = np.concatenate([kp.astype(np.float16).astype(np.float32), ck[None]], 0)
    vf = np.concatenate([vp.astype(np.float16).astype(np.float32), cvv[None]], 0)
    s = np.einsum("bhd,tbhd->bht", q, kf) / math.sqrt(D)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bht,tbhv->bhv", p, vf)
    assert np.max(np.abs(got - want)) <= 1e-5


# ------------------------------------------------------------------ absorbed MLA
def q8_0_block(scale_bits, quant):
    return np.concatenate([np.array([scale_bits & 0xFF, scale_bits >> 8], np.uint8), np.full(32, quant & 0xFF, np.uint8)])


def test_absorbed_mla_sequence_matches_causal_q8_reference():
    # metal/q2.rs:8214-8390, tolerance 2e-4: K_b -> scores over latent+rope -> softmax -> sum p*latent -> V_b
    B, T, H, qn, R, L, Dv, past, P = 1, 3, 2, 32, 8, 32, 32, 2, 4
    q_no = ((np.arange(T * H * qn) - 17.0) * 0.01).astype(np.float32)
    q_rope = ((np.arange(T * H * R) + 1.0) * -0.015).astype(np.float32)
    cur_lat = ((np.arange(T * L) - 9.0) * 0.02).astype(np.float32)
    cur_rope = ((np.arange(T * R) + 2.0) * 0.025).astype(np.float32)
    paged_lat = np.zeros(P * L, np.float32)
    paged_rope = np.zeros(P * R, np.float32)
    for t in range(past):
        paged_lat[t * L:(t + 1) * L] = (t * L + np.arange(L) + 3) * np.float32(0.007)
        paged_rope[t * R:(t + 1) * R] = (t * R + np.arange(R) + 1) * np.float32(-0.011)
    k_b = np.concatenate([q8_0_block(0x2C00, ((h + o) % 5) - 2) for h in range(H) for o in range(L)])
    v_b = np.concatenate([q8_0_block(0x2800, ((h * 2 + o) % 7) - 3) for h in range(H) for o in range(Dv)])

    q_lat = orc.q8_0_heads_matvec(k_b, q_no, H, qn, L)           # [T,H,L]
    ctx = orc.mla_absorbed_f32(q_lat, q_rope, paged_lat, cur_lat, paged_rope, cur_rope, B, H, T, past, P, L, R, qn + R)
    got = orc.q8_0_heads_matvec(v_b, ctx, H, L, Dv).reshape(T, H, Dv)

    # independent numpy statement of the test's expected value
    kscale, vscale = float(np.array([0x2C00], np.uint16).view(np.float16)[0]), float(np.array([0x2800], np.uint16).view(np.float16)[0])
    want = np.zeros((T, H, Dv), np.float32)
    lat_all = np.concatenate([paged_lat.reshape(P, L)[:past], cur_lat.reshape(T, L)])
    rope_all = np.concatenate([paged_rope.reshape(P, R)[:past], cur_rope.reshape(T, R)])
    for t in range(T):
        for h in range(H):
            kq = np.array([((h + o) % 5) - 2 for o in range(L)], np.float32) * kscale
            ql = kq * q_no.reshape(T, H, qn)[t, h].sum()          # constant-quant rows: every weight in a row is equal
            n = past + t + 1
            s = (lat_all[:n] @ ql + rope_all[:n] @ q_rope.reshape(T, H, R)[t, h]) / math.sqrt(qn + R)
            p = np.exp(s - s.max())
            p /= p.sum()
            c = p @ lat_all[:n]
            vq = np.array([((h * 2 + o) % 7) - 3 for o in range(Dv)], np.float32) * vscale
            want[t, h] = vq * c.sum()
    assert np.max(np.abs(got - want)) <= 2e-4

    # the fused-row / page-table extension reproduces the f32 identity-page kernel when values are fp16-exact
    q_cat = np.concatenate([q_lat.reshape(B, T, H, L), q_rope.reshape(B, T, H, R)], -1)
    q_cat = orc.round_f16(q_cat)
    rows = orc.round_f16(np.concatenate([cur_lat.reshape(B, T, L), cur_rope.reshape(B, T, R)], -1))
    pool = np.zeros((3, P, L + R), np.uint16)
    page_table = np.array([[2, 0]], np.int32)
    pl = orc.round_f16(paged_lat).reshape(P, L)
    pr = orc.round_f16(paged_rope).reshape(P, R)
    pool[2] = np.concatenate([pl, pr], -1).astype(np.float16).view(np.uint16)
    got2 = orc.mla_absorbed_paged(q_cat, rows, pool, page_table, np.array([past], np.int32), P, L, R,
                                  1.0 / math.sqrt(qn + R))
    ref2 = orc.mla_absorbed_f32(q_cat[..., :L], q_cat[..., L:], pl, rows[..., :L], pr, rows[..., L:], B, H, T, past, P,
                                L, R, qn + R)
    assert np.max(np.abs(got2 - ref2)) <= 1e-6
    # rows 2,3 of the first page and row 0 of the second page now hold the appended tokens
    assert np.array_equal(pool[2, 2].view(np.float16).astype(np.float32), rows[0, 0])
    assert np.array_equal(pool[0, 0].view(np.float16).astype(np.float32), rows[0, 2])


# ------------------------------------------------------------------ paged extension vs ring kernel
def test_paged_gqa_equals_ring_under_any_page_table():
    B, T0, Hq, Hkv, D, P = 2, 21, 12, 2, 128, 16
    q = orc.fill_normal((B, T0 + 1, Hq, D), 11)
    k = orc.fill_normal((B, T0 + 1, Hkv, D), 12)
    v = orc.fill_normal((B, T0 + 1, Hkv, D), 13)
    cap = 64
    outs = []
    for paged in (False, True):
        if paged:
            pages_per_seq = cap // P
            perm = orc.permutation(B * pages_per_seq + 5, 99)
            pt = perm[:B * pages_per_seq].reshape(B, pages_per_seq)
            kp = np.zeros((B * pages_per_seq + 5, Hkv, P, D), np.uint16)
            vp = np.zeros_like(kp)
            past0 = np.zeros(B, np.int32)
            orc.gqa_paged_attention(q[:, :T0], k[:, :T0], v[:, :T0], None, kp, vp, pt, past0, P)
            o = orc.gqa_paged_attention(q[:, T0:], k[:, T0:], v[:, T0:], None, kp, vp, pt, past0 + T0, P)
            lin = orc.linearize_paged(kp, pt, T0 + 1, P)  # [B,Hkv,T,D]
            assert np.array_equal(lin.view(np.float16), np.transpose(k, (0, 2, 1, 3)).astype(np.float16))
        else:
            ck = np.zeros((B, cap, Hkv, D), np.uint16)
            cv = np.zeros_like(ck)
            # the ring kernel hard-wires 8 KV heads only through its constants; the oracle takes kv_heads
            from oracle.pyoracle import lib, _p
            import ctypes as C
            o = np.empty((B, 1, Hq, D), np.float32)
            tmp = np.empty((B, T0, Hq, D), np.float32)
            qa, ka, va = [np.ascontiguousarray(a[:, :T0]) for a in (q, k, v)]
            lib().orc_gqa_ring_attention(_p(qa), _p(ka), _p(va), None, _p(ck), _p(cv), _p(tmp), B, Hq, Hkv, D, T0, 0, 0, cap, 0, 1)
            qb, kb, vb = [np.ascontiguousarray(a[:, T0:]) for a in (q, k, v)]
            lib().orc_gqa_ring_attention(_p(qb), _p(kb), _p(vb), None, _p(ck), _p(cv), _p(o), B, Hq, Hkv, D, 1, T0, T0, cap, 0, 1)
        outs.append(o)
    assert np.array_equal(outs[0], outs[1])


def test_q8_row_codec_round_trips_with_bounded_error():
    """crates/cache/src/cold_kv.rs:1903-1911: tensor(2, -1.0) = [1,2,2,32] with values -1 + i/10 round-trips within
    0.08 and the payload is smaller than the f32 tensor; plus the layout facts of encode_q8_rows (:1624-1655)."""
    src = (-1.0 + np.arange(1 * 2 * 2 * 32, dtype=np.float32) / np.float32(10.0)).reshape(-1, 32)
    payload = orc.q8_rows_encode(src)
    back = orc.q8_rows_decode(payload, 32)
    assert np.max(np.abs(back - src)) <= 0.08
    assert payload.size < src.size * 4 and payload.shape == (4, 36)
    # scale = max|x| / 127 as little-endian f32, the extreme value maps to +-127
    scale = payload[:, :4].copy().view("<f4").reshape(-1)
    assert np.array_equal(scale, (np.abs(src).max(axis=1) / np.float32(127.0)).astype(np.float32))
    assert np.all(np.abs(payload[:, 4:].view(np.int8)).max(axis=1) == 127)
    # an all-zero row has scale 1.0 and zero quants; halves round away from zero
    z = orc.q8_rows_encode(np.array([[0, 0, 0, 0], [127, 0.5, -0.5, 2.5]], np.float32))
    assert z[0].tolist() == [0, 0, 128, 63, 0, 0, 0, 0]
    assert z[1, 4:].view(np.int8).tolist() == [127, 1, -1, 3]


def test_dsa_topk_ordering_rule():
    """dsa_precedes (crates/backend/src/metal/kernels/dsa_kernels.metal:182-196): higher score first, equal scores by
    lower id, invalid ids last."""
    scores = np.array([[0.5, 2.0, 2.0, -1.0, 0.5, 0.0, -0.0]], np.float32)
    assert orc.dsa_topk(scores, 5)[0].tolist() == [1, 2, 0, 4, 5]
    assert orc.dsa_topk(scores, 9)[0].tolist() == [1, 2, 0, 4, 5, 6, 3, 0xFFFFFFFF, 0xFFFFFFFF]


def test_dsa_scores_formula():
    """dsa_scores_f32_kernel (dsa_kernels.metal:137-176) on a closed-form case: one-hot queries pick key columns."""
    q = np.zeros((1, 2, 4), np.float32)
    q[0, 0, 0] = 1.0
    q[0, 1, 1] = 2.0
    w = np.array([[0.5, 0.25]], np.float32)
    past = np.array([[[4.0, -1.0, 9, 9], [-2.0, 3.0, 9, 9]]], np.float32)
    cur = np.array([[1.0, 1.0, 9, 9]], np.float32)
    # scale 1/sqrt(4) = 0.5: token0: 0.5*relu(2) + 0.25*relu(-1) = 1.0; token1: 0.5*relu(-1) + 0.25*relu(3) = 0.75;
    # current: 0.5*relu(0.5) + 0.25*relu(1) = 0.5
    assert np.allclose(orc.dsa_scores(q, w, past, cur), [[1.0, 0.75, 0.5]])


def test_fp8_e4m3fn_codec_matches_the_published_format():
    """The FP8 codec restatement (fp8_attention_kernels.metal:11-54) against the E4M3FN format itself: known codes,
    a round trip of every code, saturation and NaN handling, and torch's own float8_e4m3fn cast for in-range values."""
    torch = pytest.importorskip("torch")
    dec = orc.fp8_e4m3fn_decode(np.arange(256, dtype=np.uint8))
    assert dec[0x38] == 1.0 and dec[0x7E] == 448.0 and dec[0x08] == 2.0 ** -6 and dec[0x01] == 2.0 ** -9
    assert dec[0x7F] == 0.0 and dec[0xFF] == 0.0 and dec[0xB8] == -1.0
    codes = np.array([c for c in range(256) if c not in (0x7F, 0xFF, 0x80)], np.uint8)
    assert np.array_equal(orc.fp8_e4m3fn_encode(dec[codes]), codes)
    special = np.array([np.nan, 0.0, -0.0, 1e9, -1e9, 464.0, 2.0 ** -10, 3 * 2.0 ** -10], np.float32)
    assert orc.fp8_e4m3fn_encode(special).tolist() == [0, 0, 0, 0x7E, 0xFE, 0x7E, 0, 2]
    x = np.concatenate([orc.fill_normal((50000,), 0xF8000 + 1500, 4.0, False),
                        orc.fill_normal((50000,), 0xF8000 + 1501, 0.02, False)]).astype(np.float32)
    x = x[(np.abs(x) <= 448) & (x != 0)]
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = orc.fp8_e4m3fn_encode(x)
    # torch keeps the sign of values that round to zero; the reference encoder does too (sign | 0)
    assert np.array_equal(got, want)


def test_dsa_decode_topk_matches_the_reference_known_answers():
    """dsa_decode_topk_device_matches_expected_ranking_when_metal_available (crates/backend/src/backend.rs:10835):
    hidden (sqrt 2, 0, 0, 0), two heads of two dims, three past keys and the current one -> ids [2, 3]; and
    layer_norm_last_dim_applies_weight_and_bias (crates/model/src/indexer.rs:633)."""
    hidden = np.array([[[math.sqrt(2.0), 0.0, 0.0, 0.0]]], np.float32)
    q_raw = np.array([[[1.0, 0.0, 0.0, 1.0]]], np.float32)
    past = np.array([[[1.0, 0.0], [0.0, 1.0], [2.0, 0.0]]], np.float32)
    cur = np.array([[[0.0, 2.0]]], np.float32)
    proj = np.array([[1.0, 1.0], [0.0, 0.0], [0.0, 0.0], [0.0, 0.0]], np.float32)
    ids = orc.dsa_decode_topk(hidden, q_raw, past, cur, proj, 2, 2, 2, 0, 10000.0, 2)
    assert ids.tolist() == [[2, 3]]
    key = orc.dsa_index_key(np.array([[[1.0, 3.0]]], np.float32), np.array([2.0, 2.0], np.float32),
                            np.array([0.5, -0.5], np.float32), 0, 0, 10000.0, 1e-6)
    assert abs(key[0, 0, 0] - -1.499999) < 1e-4 and abs(key[0, 0, 1] - 1.499999) < 1e-4
    # the rotation writes halves: pair (x0, x1) at position 1 with freq 1 -> (x0 cos1 - x1 sin1, x1 cos1 + x0 sin1)
    r = orc.dsa_rotate_interleaved(np.array([1.0, 2.0, 3.0, 4.0, 9.0], np.float32), 4, 1, 10000.0)
    c0, s0, f1 = math.cos(1.0), math.sin(1.0), 1.0 / math.sqrt(10000.0)
    want = [1 * c0 - 2 * s0, 3 * math.cos(f1) - 4 * math.sin(f1), 2 * c0 + 1 * s0, 4 * math.cos(f1) + 3 * math.sin(f1), 9.0]
    assert np.allclose(r, want, atol=1e-6)


# ---------------------------------------------------------------------------------------------------------------
# FP8 E4M3FN cache: crates/backend/src/metal/fp8_attention.rs tests, replayed on the paged oracle
# ---------------------------------------------------------------------------------------------------------------
def test_fp8_codec_c_restatement_equals_the_numpy_statement():
    bits = np.arange(256, dtype=np.uint8)
    assert np.array_equal(orc.fp8_codec_c(bits=bits).view(np.uint32), orc.fp8_e4m3fn_decode(bits).view(np.uint32))
    grid = np.sort(orc.fp8_e4m3fn_decode(np.arange(127, dtype=np.uint8)))
    x = np.concatenate([grid, (grid[:-1] + grid[1:]) / 2, -grid, orc.fill_normal((4000,), 99, 3.0, False),
                        np.array([0.0, -0.0, np.nan, 448.0, 449.0, 1e9, -1e9, 464.0, 1.1, 2.0 ** -10, 1e-30], np.float32)])
    assert np.array_equal(orc.fp8_codec_c(values=x), orc.fp8_e4m3fn_encode(x))
    assert orc.fp8_codec_c(values=[1.1])[0] == 0x39 and orc.fp8_codec_c(bits=[0x39])[0] == np.float32(1.125)


def _fp8_paged(pages, P=16, Hkv=8, D=128):
    return (np.zeros((pages, Hkv, P, D), np.uint8), np.zeros((pages, Hkv, P, D), np.uint8),
            np.arange(pages, dtype=np.int32)[None])


def test_fp8_global_prefill_append_and_decode():
    """fp8_attention.rs:489-561: zero queries, values 1.1 and 3.0 prefilled (causal means 1.1 and 2.05), then a decode
    with value 5.0: the two cached values come back through FP8 (1.1 -> 1.125), the current one is f32."""
    Hq, Hkv, D = 48, 8, 128
    kp, vp, pt = _fp8_paged(2)
    q = np.zeros((1, 2, Hq, D), np.float32)
    k = np.zeros((1, 2, Hkv, D), np.float32)
    v = np.zeros((1, 2, Hkv, D), np.float32)
    v[0, 0], v[0, 1] = 1.1, 3.0
    gate = np.zeros((1, 2, Hq), np.float32)
    out = orc.gqa_paged_attention_fp8(q, k, v, gate, kp, vp, 1.0, 1.0, pt, [0], 16)
    ln2 = np.float32(np.log(2.0))
    assert np.abs(out[0, 0] - 1.1 * ln2).max() <= 1e-4 and np.abs(out[0, 1] - 2.05 * ln2).max() <= 1e-4
    out = orc.gqa_paged_attention_fp8(q[:, :1], k[:, :1], np.full((1, 1, Hkv, D), 5.0, np.float32), gate[:, :1], kp, vp,
                                      1.0, 1.0, pt, [2], 16)
    assert np.abs(out - (1.125 + 3.0 + 5.0) / 3.0 * ln2).max() <= 1e-4
    assert vp[0, 0, 0, 0] == 0x39 and vp[0, 0, 2, 0] == orc.fp8_e4m3fn_encode(np.float32([5.0]))[0]


def test_fp8_sliding_window_over_a_full_ring():
    """fp8_attention.rs:563-625: 511 cached rows of value 1.0 (byte 0x38), window 512, two tokens 3.0 and 5.0, then a
    decode of 7.0: 514/512, 518/512 and 524/512 times softplus(0)."""
    Hq, Hkv, D, W = 72, 8, 128, 512
    kp, vp, pt = _fp8_paged(40)
    for t in range(511):
        vp[t // 16, :, t % 16] = 0x38
    q = np.zeros((1, 2, Hq, D), np.float32)
    k = np.zeros((1, 2, Hkv, D), np.float32)
    v = np.zeros((1, 2, Hkv, D), np.float32)
    v[0, 0], v[0, 1] = 3.0, 5.0
    gate = np.zeros((1, 2, Hq), np.float32)
    ln2 = np.float32(np.log(2.0))
    out = orc.gqa_paged_attention_fp8(q, k, v, gate, kp, vp, 1.0, 1.0, pt, [511], 16, sliding_window=W)
    assert np.abs(out[0, 0] - 514.0 / 512.0 * ln2).max() <= 1e-4 and np.abs(out[0, 1] - 518.0 / 512.0 * ln2).max() <= 1e-4
    out = orc.gqa_paged_attention_fp8(q[:, :1], k[:, :1], np.full((1, 1, Hkv, D), 7.0, np.float32), gate[:, :1], kp, vp,
                                      1.0, 1.0, pt, [513], 16, sliding_window=W)
    assert np.abs(out - 524.0 / 512.0 * ln2).max() <= 1e-4


def test_fp8_sliding_prefill_longer_than_the_window():
    """fp8_attention.rs:429-487: 513 tokens of value 2.0 (the first one 100.0) through a 512 window: the last row sees
    only 2.0; a decode of 4.0 then sees 511 x 2.0 and itself."""
    Hq, Hkv, D, W, T = 72, 8, 128, 512, 513
    kp, vp, pt = _fp8_paged(40)
    q = np.zeros((1, T, Hq, D), np.float32)
    k = np.zeros((1, T, Hkv, D), np.float32)
    v = np.full((1, T, Hkv, D), 2.0, np.float32)
    v[0, 0] = 100.0
    gate = np.zeros((1, T, Hq), np.float32)
    ln2 = np.float32(np.log(2.0))
    out = orc.gqa_paged_attention_fp8(q, k, v, gate, kp, vp, 1.0, 1.0, pt, [0], 16, sliding_window=W)
    assert abs(out[0, T - 1, 0, 0] - 2.0 * ln2) < 1e-3
    out = orc.gqa_paged_attention_fp8(q[:, :1], k[:, :1], np.full((1, 1, Hkv, D), 4.0, np.float32), gate[:, :1], kp, vp,
                                      1.0, 1.0, pt, [T], 16, sliding_window=W)
    assert abs(out[0, 0, 0, 0] - ((W - 1) * 2.0 + 4.0) / W * ln2) < 1e-3


# ---------------------------------------------------------------------------------------------------------------
# selected-row attention over expanded heads: metal/attention.rs:2413-2740, closed-form inputs, tolerance 1e-5
# ---------------------------------------------------------------------------------------------------------------
def _ramp(n, div):
    return ((np.arange(n, dtype=np.float32) + np.float32(1.0)) / np.float32(div)).astype(np.float32)


def numpy_selected_attention(q, sel_k, sel_v, cur_k, cur_v, include_current=True):
    """Independent statement (cpu_attention_scores / causal_softmax / values, metal/attention.rs): float64 throughout."""
    B, H, T, D = q.shape
    S = 0 if sel_k is None else sel_k.shape[2]
    out = np.zeros((B, H, T, cur_v.shape[3]))
    for b in range(B):
        for h in range(H):
            for t in range(T):
                ks = [sel_k[b, h]] if S else []
                vs = [sel_v[b, h]] if S else []
                if include_current:
                    ks.append(cur_k[b, h, :t + 1])
                    vs.append(cur_v[b, h, :t + 1])
                K, V = np.concatenate(ks).astype(np.float64), np.concatenate(vs).astype(np.float64)
                s = K @ q[b, h, t].astype(np.float64) / np.sqrt(D)
                p = np.exp(s - s.max())
                out[b, h, t] = (p / p.sum()) @ V
    return out.astype(np.float32)


def selected_attention_cases():
    B, H, D, Dv = 1, 2, 4, 3
    yield ("decode, 4 selected + current (attention.rs:2413)", _ramp(B * H * D, 10).reshape(B, H, 1, D),
           _ramp(B * H * 4 * D, 20).reshape(B, H, 4, D), _ramp(B * H * 4 * Dv, 30).reshape(B, H, 4, Dv),
           _ramp(B * H * D, 40).reshape(B, H, 1, D), _ramp(B * H * Dv, 50).reshape(B, H, 1, Dv), True)
    yield ("sequence, 3 past + 8 rows (attention.rs:2564)", _ramp(B * H * 8 * D, 10).reshape(B, H, 8, D),
           _ramp(B * H * 3 * D, 20).reshape(B, H, 3, D), _ramp(B * H * 3 * Dv, 30).reshape(B, H, 3, Dv),
           _ramp(B * H * 8 * D, 40).reshape(B, H, 8, D), _ramp(B * H * 8 * Dv, 50).reshape(B, H, 8, Dv), True)
    yield ("current-only prefill chunk (attention.rs:2668)", _ramp(B * H * 8 * D, 10).reshape(B, H, 8, D), None, None,
           _ramp(B * H * 8 * D, 20).reshape(B, H, 8, D), _ramp(B * H * 8 * Dv, 30).reshape(B, H, 8, Dv), True)
    yield ("decode without the current token", _ramp(B * H * D, 10).reshape(B, H, 1, D),
           _ramp(B * H * 4 * D, 20).reshape(B, H, 4, D), _ramp(B * H * 4 * Dv, 30).reshape(B, H, 4, Dv),
           _ramp(B * H * D, 40).reshape(B, H, 1, D), _ramp(B * H * Dv, 50).reshape(B, H, 1, Dv), False)


def test_selected_attention_reference_cases():
    for name, q, sk, sv, ck, cv, inc in selected_attention_cases():
        got = orc.selected_attention(q, sk, sv, ck, cv, inc)
        assert np.abs(got - numpy_selected_attention(q, sk, sv, ck, cv, inc)).max() <= 1e-5, name
