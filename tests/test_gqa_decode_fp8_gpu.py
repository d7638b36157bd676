"""GPU parity: fused RoPE + append into FP8 E4M3FN pages and the paged GQA decode that reads those pages directly,
against the oracle (fp8_attention_kernels.metal:70-263 restated over pages), through the C ABI."""
import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0, assert_close, scatter_pages

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from inferno_b200 import CudaBackend
    b = CudaBackend(0)
    yield b
    b.device_flush()
    b.close()


def dev(be, a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(be.device)
    return t if dtype is None else t.to(dtype)


def fill_fp8_pools(lens, pt, num_pages, Hkv, P, D, seed, key_scale, value_scale):
    """Pools holding lens[b] cached rows per sequence: N(0,1) values through the reference's encoder."""
    kp = np.zeros((num_pages, Hkv, P, D), np.uint8)
    vp = np.zeros_like(kp)
    for b, n in enumerate(lens):
        if n == 0:
            continue
        k = orc.fp8_e4m3fn_encode(orc.fill_normal((n, Hkv, D), seed + 1000 * b + 1) / np.float32(key_scale))
        v = orc.fp8_e4m3fn_encode(orc.fill_normal((n, Hkv, D), seed + 1000 * b + 2) / np.float32(value_scale))
        for s in range((n + P - 1) // P):
            t0, t1 = s * P, min(n, (s + 1) * P)
            kp[pt[b, s], :, :t1 - t0] = np.transpose(k[t0:t1], (1, 0, 2))
            vp[pt[b, s], :, :t1 - t0] = np.transpose(v[t0:t1], (1, 0, 2))
    return kp, vp


def run_case(be, past, Hq, Hkv, chunk, window, use_gate, key_scale, value_scale, seed):
    D, P = 128, 16
    B = len(past)
    pages = [(n + 1 + P - 1) // P for n in past]
    num_pages = sum(pages) + 9
    pt = scatter_pages(pages, num_pages, seed)
    kp, vp = fill_fp8_pools(past, pt, num_pages, Hkv, P, D, seed, key_scale, value_scale)
    q = orc.fill_normal((B, 1, Hq, D), seed + 11)
    k = orc.fill_normal((B, 1, Hkv, D), seed + 12)
    v = orc.fill_normal((B, 1, Hkv, D), seed + 13)
    gate = orc.fill_normal((B, 1, Hq), seed + 14, 2.0, False) if use_gate else None
    inv = orc.default_inv_freq(500000.0, 64)
    pos = np.array(past, np.int32)
    pool = be.prepare_kv_pool_fp8(num_pages, P, Hkv, key_scale, value_scale)
    pool.k.copy_(dev(be, kp))
    pool.v.copy_(dev(be, vp))
    want = orc.gqa_paged_attention_fp8(orc.qk_norm_rope(q, None, inv, 64, 0, positions=pos),
                                       orc.qk_norm_rope(k, None, inv, 64, 0, positions=pos), v, gate, kp, vp, key_scale,
                                       value_scale, pt, past, P, sliding_window=window)
    rope = be.prepare_rope_table(inv, 64, 1.0)
    table = be.page_table(pt, past)
    q16, k16, v16 = be.rope_append_gqa_fp8(dev(be, q, torch.float16), dev(be, k, torch.float16), dev(be, v, torch.float16),
                                            rope, pool, table)
    out = be.gqa_decode_paged_fp8(q16[:, 0].contiguous(), k16[:, 0].contiguous(), v16[:, 0].contiguous(), pool, table,
                                  max_len=max(past) + 1, split_chunk=chunk, sliding_window=window,
                                  gate=dev(be, gate[:, 0]) if use_gate else None)
    be.device_flush()
    # the append is byte work: V pages are bit-exact; roped K may differ by one code where cosf/sinf differ from libm
    assert np.array_equal(pool.v.cpu().numpy(), vp)
    kd = pool.k.cpu().numpy()
    assert (kd != kp).mean() < 0.002
    assert_close(out.cpu().numpy(), want[:, 0], f"fp8 decode past={past}")
    return out


@pytest.mark.parametrize("past,Hq,Hkv,chunk,window,use_gate,ks,vs", [
    ([0], 48, 8, 512, 0, False, 1.0, 1.0),                 # nothing cached: the output is the current value
    ([1, 15, 16, 17, 1000], 48, 8, 512, 0, True, 0.5, 0.25),  # page edges, ragged batch, gate, scales != 1
    ([700, 63, 513], 12, 2, 64, 0, False, 0.037, 0.021),   # many chunks, arbitrary scales
    ([600, 2000], 64, 8, 128, 512, True, 1.0, 2.0),        # sliding window
    ([300], 72, 8, 256, 0, False, 1.0, 1.0),               # 9 heads per group
    ([5000, 2048, 4097], 48, 8, 512, 0, False, 0.05, 0.05),  # runs of chunks over several CTAs
])
def test_fp8_decode_matches_oracle(be, past, Hq, Hkv, chunk, window, use_gate, ks, vs):
    run_case(be, past, Hq, Hkv, chunk, window, use_gate, ks, vs, SEED0 + 1500 + len(past) + Hq)


def test_fp8_config3_full_size(be):
    """The batch-32 decode configuration (48 / 8 heads, contexts U{1024..16384}, chunk 512, 16-token pages) over FP8
    pages: half the bytes of the fp16 form, same oracle tolerance."""
    from bench import decode_lens
    run_case(be, [int(n) - 1 for n in decode_lens(0, 32)], 48, 8, 512, 0, False, 0.03, 0.03, SEED0 + 1600)


def test_fp8_reference_known_answers(be):
    """fp8_attention.rs:489-561 through the CUDA path: values 1.1 and 3.0 cached through FP8 (1.1 -> 1.125), decode of
    5.0 with zero queries and zero gate: (1.125 + 3 + 5) / 3 * ln 2, tolerance 1e-4 as in the reference."""
    Hq, Hkv, D, P = 48, 8, 128, 16
    pool = be.prepare_kv_pool_fp8(4, P, Hkv, 1.0, 1.0)
    pt = np.array([[2, 0, 3, 1]], np.int32)
    z = lambda *s: torch.zeros(s, dtype=torch.float32, device=be.device)
    v = z(1, 2, Hkv, D)
    v[0, 0], v[0, 1] = 1.1, 3.0
    be.rope_append_gqa_fp8(z(1, 2, Hq, D), z(1, 2, Hkv, D), v, None, pool, be.page_table(pt, [0]))
    q16, k16, v16 = be.rope_append_gqa_fp8(z(1, 1, Hq, D), z(1, 1, Hkv, D), torch.full((1, 1, Hkv, D), 5.0, device=be.device),
                                            None, pool, be.page_table(pt, [2]))
    out = be.gqa_decode_paged_fp8(q16[:, 0].contiguous(), k16[:, 0].contiguous(), v16[:, 0].contiguous(), pool,
                                  be.page_table(pt, [2]), max_len=3, gate=z(1, Hq))
    be.device_flush()
    assert np.abs(out.cpu().numpy() - (1.125 + 3.0 + 5.0) / 3.0 * np.log(2.0)).max() <= 1e-4
    assert pool.v.cpu().numpy()[2, 0, 0, 0] == 0x39


def test_fp8_host_validation(be):
    from inferno_b200 import InfernoError
    with pytest.raises(InfernoError) as e:
        be.prepare_kv_pool_fp8(4, 16, 8, 0.0, 1.0)
    assert e.value.kind == "Config"
    pool = be.prepare_kv_pool_fp8(4, 16, 2, 1.0, 1.0)
    q = torch.zeros((1, 8, 128), dtype=torch.float16, device=be.device)
    kv = torch.zeros((1, 2, 128), dtype=torch.float16, device=be.device)
    with pytest.raises(InfernoError) as e:  # 40 cached rows + the current one do not fit max_len 40
        be.gqa_decode_paged_fp8(q, kv, kv, pool, be.page_table([[0, 1, 2]], [40]), max_len=40)
    assert e.value.kind == "ShapeMismatch"
    be.device_flush()
