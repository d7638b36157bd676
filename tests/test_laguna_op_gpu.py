"""GPU parity of the drop-in operators, on the reference's own test cases.

inf_laguna_gated_gqa_f16_attention replays crates/backend/src/metal/f16_attention.rs:708-767 (ln 2 identities),
:792-842 (8-token prefill, 48 heads) and :955-1075 (decode after a 36-token prefill; 599 tokens under the
512-token window), with the reference's tolerances, over a paged cache instead of its ring.
inf_paged_decode_attention_resident replays the resident F16 paged decode (metal/attention.rs:2742-2859)."""
import math

import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import scatter_pages

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

D, KV = 128, 8


@pytest.fixture(scope="module")
def be():
    from inferno_b200 import CudaBackend
    b = CudaBackend(0)
    yield b
    b.device_flush()
    b.close()


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(be.device)


def patterned(n, period, center, divisor):
    idx = np.arange(n)
    return ((idx % period).astype(np.float32) - np.float32(center)) / np.float32(divisor)


def test_ln2_identities(be):
    Hq, P = 48, 16
    pool = be.prepare_kv_pool(4, P, KV, D)
    pt = np.array([[2, 0]], np.int32)
    q = np.zeros((1, 2, Hq, D), np.float32)
    k = np.zeros((1, 2, KV, D), np.float32)
    v = np.ones((1, 2, KV, D), np.float32)
    v[0, 1] = 3.0
    gate = np.zeros((1, 2, Hq), np.float32)
    out = be.laguna_gated_gqa_f16_attention_device(dev(be, q), dev(be, k), dev(be, v), dev(be, gate), pool,
                                                   be.page_table(pt, [0]), max_len=4)
    be.device_flush()
    ln2 = math.log(2.0)
    o = out.cpu().numpy()
    assert abs(o[0, 0, 0, 0] - ln2) <= 1e-4 and abs(o[0, 1, 0, 0] - 2 * ln2) <= 1e-4
    out = be.laguna_gated_gqa_f16_attention_device(dev(be, q[:, :1]), dev(be, k[:, :1]),
                                                   dev(be, np.full((1, 1, KV, D), 5.0)), dev(be, gate[:, :1]), pool,
                                                   be.page_table(pt, [2]), max_len=4)
    be.device_flush()
    assert abs(out.cpu().numpy()[0, 0, 0, 0] - 3 * ln2) <= 1e-4


def test_prefill_matches_nonuniform_cpu_reference(be):
    T, Hq, P = 8, 48, 16
    q = patterned(T * Hq * D, 17, 8, 16.0).reshape(1, T, Hq, D)
    k = patterned(T * KV * D, 13, 6, 16.0).reshape(1, T, KV, D)
    v = patterned(T * KV * D, 11, 5, 8.0).reshape(1, T, KV, D)
    gate = patterned(T * Hq, 7, 3, 10.0).reshape(1, T, Hq)
    pool = be.prepare_kv_pool(3, P, KV, D)
    out = be.laguna_gated_gqa_f16_attention_device(dev(be, q), dev(be, k), dev(be, v), dev(be, gate), pool,
                                                   be.page_table([[1]], [0]), max_len=T)
    be.device_flush()
    want = orc.test_cpu_gqa(q, k, v, gate, Hq, KV, D)
    # the reference tolerance is max(5e-4, 5e-4|x|) for an all-f32 kernel; here Q and the chunk's K are rounded to
    # fp16 on their way in, so the stated fp16 tolerance applies
    err = np.abs(out.cpu().numpy()[0] - want)
    assert np.all(err <= 2e-3 + 1e-2 * np.abs(want)), err.max()


@pytest.mark.parametrize("sliding,q_heads,tokens", [(False, 48, 37), (True, 64, 600), (True, 72, 600)])
def test_decode_step_matches_nonuniform_cpu_reference(be, sliding, q_heads, tokens):
    P = 16
    q = patterned(tokens * q_heads * D, 17, 8, 16.0).reshape(1, tokens, q_heads, D)
    k = patterned(tokens * KV * D, 13, 6, 16.0).reshape(1, tokens, KV, D)
    v = patterned(tokens * KV * D, 11, 5, 8.0).reshape(1, tokens, KV, D)
    gate = patterned(tokens * q_heads, 7, 3, 10.0).reshape(1, tokens, q_heads)
    window = 512 if sliding else 0
    pages = (tokens + P - 1) // P
    pt = scatter_pages([pages], pages + 3, 77)
    pool = be.prepare_kv_pool(pages + 3, P, KV, D)
    prefill = tokens - 1
    be.laguna_gated_gqa_f16_attention_device(dev(be, q[:, :prefill]), dev(be, k[:, :prefill]), dev(be, v[:, :prefill]),
                                             dev(be, gate[:, :prefill]), pool, be.page_table(pt, [0]), max_len=tokens,
                                             sliding_window=window)
    out = be.laguna_gated_gqa_f16_attention_device(dev(be, q[:, prefill:]), dev(be, k[:, prefill:]),
                                                   dev(be, v[:, prefill:]), dev(be, gate[:, prefill:]), pool,
                                                   be.page_table(pt, [prefill]), max_len=tokens, sliding_window=window)
    be.device_flush()
    want = orc.test_cpu_gqa(q, k, v, gate, q_heads, KV, D, window, last_only=True)
    got = out.cpu().numpy()[0, 0]
    assert np.all(np.abs(got - want) <= np.maximum(2e-3, np.abs(want) * 2e-3))  # the reference tolerance


@pytest.mark.parametrize("B,H,Dk,Dv,P,past", [
    (2, 64, 256, 256, 128, 300),    # the key-split kernel (rows through the shared-memory ring), two splits
    (1, 64, 256, 256, 64, 4095),    # the GLM expanded layout at the reference kernel's limit of 4096 keys
    (3, 5, 192, 128, 16, 1000),     # 192 / 128 dims, ragged last split
    (2, 4, 96, 32, 16, 700),        # dims that are not multiples of 64: the one-CTA-per-row kernel
    (1, 8, 256, 256, 128, 100),     # too few keys to split
    (2, 8, 128, 128, 24, 500),      # pages that do not hold a multiple of 16 keys: the threads load the rows themselves
    (1, 3, 128, 128, 16, 2000),     # one key per 16-key page tile short of a multiple: ragged last tile of the ring
])
def test_glm_paged_f16_decode_sizes(be, B, H, Dk, Dv, P, past):
    rng = np.random.default_rng(past)
    pages = (past + P - 1) // P
    pk = (rng.standard_normal((pages, B, H, P, Dk)) * 0.5).astype(np.float16)
    pv = (rng.standard_normal((pages, B, H, P, Dv)) * 0.5).astype(np.float16)
    q = rng.standard_normal((B, H, Dk)).astype(np.float32)
    ck = rng.standard_normal((B, H, Dk)).astype(np.float32)
    cv = rng.standard_normal((B, H, Dv)).astype(np.float32)
    want = orc.paged_decode_mha_f16(q, pk.view(np.uint16), ck, pv.view(np.uint16), cv, past, P)
    out = be.paged_decode_attention_resident_device(dev(be, q), torch.from_numpy(pk).to(be.device), dev(be, ck),
                                                    torch.from_numpy(pv).to(be.device), dev(be, cv), past, P)
    be.device_flush()
    assert np.max(np.abs(out.cpu().numpy() - want)) <= 2e-5


def test_glm_paged_f16_decode_matches_oracle(be):
    B, H, Dk, Dv, P, past = 2, 64, 256, 256, 128, 300
    rng = np.random.default_rng(11)
    pages = (past + P - 1) // P
    pk = (rng.standard_normal((pages, B, H, P, Dk)) * 0.5).astype(np.float16)
    pv = (rng.standard_normal((pages, B, H, P, Dv)) * 0.5).astype(np.float16)
    q = rng.standard_normal((B, H, Dk)).astype(np.float32)
    ck = rng.standard_normal((B, H, Dk)).astype(np.float32)
    cv = rng.standard_normal((B, H, Dv)).astype(np.float32)
    want = orc.paged_decode_mha_f16(q, pk.view(np.uint16), ck, pv.view(np.uint16), cv, past, P)
    out = be.paged_decode_attention_resident_device(dev(be, q), torch.from_numpy(pk).to(be.device), dev(be, ck),
                                                    torch.from_numpy(pv).to(be.device), dev(be, cv), past, P)
    be.device_flush()
    assert np.max(np.abs(out.cpu().numpy() - want)) <= 2e-5
    # no cached tokens: the output is the current value row
    out0 = be.paged_decode_attention_resident_device(dev(be, q), None, dev(be, ck), None, dev(be, cv), 0, P)
    be.device_flush()
    assert np.max(np.abs(out0.cpu().numpy() - cv)) <= 1e-6
