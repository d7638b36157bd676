"""GPU parity: fused RoPE + KV-append and paged GQA decode against the CPU oracle, through the C ABI."""
import math

import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0, assert_close, fill_gqa_pools, scatter_pages

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


def test_config1_rope_append_decode_bit_exact_gather(be):
    """1 sequence, 8 q / 2 kv heads, ctx 512, theta 1e4 on positions 0..511, 16-token pages under a seeded
    permutation of a 64-page pool; fp32 output."""
    B, Hq, Hkv, D, ctx, P, pool_pages = 1, 8, 2, 128, 512, 16, 64
    seed = SEED0 + 0
    q = orc.fill_normal((B, ctx, Hq, D), seed + 1)
    k = orc.fill_normal((B, ctx, Hkv, D), seed + 2)
    v = orc.fill_normal((B, ctx, Hkv, D), seed + 3)
    inv = orc.default_inv_freq(10000.0, 128)
    pt = scatter_pages([ctx // P], pool_pages, seed + 4)

    # oracle: rope, then prefill-append 511 rows, then the decode row
    q_r = orc.qk_norm_rope(q, None, inv, 128, 0)
    k_r = orc.qk_norm_rope(k, None, inv, 128, 0)
    kp = np.zeros((pool_pages, Hkv, P, D), np.uint16)
    vp = np.zeros_like(kp)
    orc.gqa_paged_attention(q_r[:, :ctx - 1], k_r[:, :ctx - 1], v[:, :ctx - 1], None, kp, vp, pt, [0], P)
    want = orc.gqa_paged_attention(q_r[:, ctx - 1:], k_r[:, ctx - 1:], v[:, ctx - 1:], None, kp, vp, pt, [ctx - 1], P)

    # CUDA path: fp16 inputs, fused rope+append for the prefix, then for the decode token, then attention
    rope = be.prepare_rope_table(inv, 128, 1.0)
    pool = be.prepare_kv_pool(pool_pages, P, Hkv, D)
    qh, kh, vh = (dev(be, a, torch.float16) for a in (q, k, v))
    be.rope_append_gqa(qh[:, :ctx - 1].contiguous(), kh[:, :ctx - 1].contiguous(), vh[:, :ctx - 1].contiguous(), rope,
                       pool, be.page_table(pt, [0]))
    q16 = be.rope_append_gqa(qh[:, ctx - 1:].contiguous(), kh[:, ctx - 1:].contiguous(), vh[:, ctx - 1:].contiguous(),
                             rope, pool, be.page_table(pt, [ctx - 1]))
    out = be.gqa_decode_paged(q16[:, 0].contiguous(), pool, be.page_table(pt, [ctx]), max_len=ctx, split_chunk=128)
    be.device_flush()

    # page/index gathering is bit-exact: V needs no arithmetic, so the pools must be identical bit for bit
    assert np.array_equal(pool.v.cpu().numpy().view(np.uint16), vp)
    # roped K: device cosf/sinf may differ from libm in the last place, so allow one fp16 ulp on a few values
    kd = pool.k.cpu().numpy().view(np.uint16).astype(np.int32)
    diff = np.abs(kd - kp.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 0.02
    # gathered logical view equals the oracle's
    lin = be.paged_kv_contiguous_device(pool.v, pool, be.page_table(pt, [ctx]), ctx).cpu().numpy().view(np.uint16)
    assert np.array_equal(lin, orc.linearize_paged(vp, pt, ctx, P))
    assert_close(out.cpu().numpy(), want[:, 0], "config 1 decode")
    # a different split must give the same answer within tolerance
    out2 = be.gqa_decode_paged(q16[:, 0].contiguous(), pool, be.page_table(pt, [ctx]), max_len=ctx, split_chunk=512)
    assert_close(out2.cpu().numpy(), want[:, 0], "config 1 decode, one chunk")


@pytest.mark.parametrize("lens,Hq,Hkv,chunk,window,use_gate", [
    ([1], 48, 8, 512, 0, False),                # a single key: softmax of one element
    ([15, 16, 17, 1000], 48, 8, 512, 0, True),  # page boundaries, ragged batch, gate
    ([700, 64, 513], 12, 2, 64, 0, False),      # many chunks
    ([600, 2000], 64, 8, 128, 512, True),       # sliding window (36 of 48 reference layers), 8 heads per group
    ([300], 72, 8, 256, 0, False),              # 9 heads per group (rows 8..15 of the MMA tile)
])
def test_decode_matches_oracle(be, lens, Hq, Hkv, chunk, window, use_gate):
    D, P = 128, 16
    seed = SEED0 + 30 + len(lens) + Hq
    B = len(lens)
    pages = [(n + P - 1) // P for n in lens]
    num_pages = sum(pages) + 7
    pt = scatter_pages(pages, num_pages, seed)
    past = [n - 1 for n in lens]
    kp, vp = fill_gqa_pools(past, pt, num_pages, Hkv, P, D, seed)
    q = orc.fill_normal((B, 1, Hq, D), seed + 11)
    k = orc.fill_normal((B, 1, Hkv, D), seed + 12)
    v = orc.fill_normal((B, 1, Hkv, D), seed + 13)
    gate = orc.fill_normal((B, 1, Hq), seed + 14, 2.0, False) if use_gate else None
    inv = orc.default_inv_freq(500000.0, 64)

    pos = np.array(past, np.int32)
    q_r = orc.qk_norm_rope(q, None, inv, 64, 0, positions=pos)
    k_r = orc.qk_norm_rope(k, None, inv, 64, 0, positions=pos)
    kp_o, vp_o = kp.copy(), vp.copy()
    want = orc.gqa_paged_attention(q_r, k_r, v, gate, kp_o, vp_o, pt, past, P, sliding_window=window)

    rope = be.prepare_rope_table(inv, 64, 1.0)
    pool = be.prepare_kv_pool(num_pages, P, Hkv, D)
    pool.k.copy_(dev(be, kp).view(torch.float16))
    pool.v.copy_(dev(be, vp).view(torch.float16))
    q16 = be.rope_append_gqa(dev(be, q, torch.float16), dev(be, k, torch.float16), dev(be, v, torch.float16), rope, pool,
                             be.page_table(pt, past))
    out = be.gqa_decode_paged(q16[:, 0].contiguous(), pool, be.page_table(pt, lens), max_len=max(lens),
                              split_chunk=chunk, sliding_window=window,
                              gate=dev(be, gate[:, 0]) if use_gate else None)
    be.device_flush()
    assert np.array_equal(pool.v.cpu().numpy().view(np.uint16), vp_o)
    assert_close(out.cpu().numpy(), want[:, 0], f"decode lens={lens}")
    # fp16 output path
    out16 = be.gqa_decode_paged(q16[:, 0].contiguous(), pool, be.page_table(pt, lens), max_len=max(lens),
                                split_chunk=chunk, sliding_window=window,
                                gate=dev(be, gate[:, 0]) if use_gate else None, out_dtype=torch.float16)
    assert_close(out16.float().cpu().numpy(), want[:, 0], "fp16 output")


def _decode_case(be, lens, Hq, Hkv, chunk, seed, theta=500000.0):
    """Fused RoPE + append of the current token, then split-KV decode, against the oracle on the same bits."""
    D, P = 128, 16
    B = len(lens)
    lens = [int(n) for n in lens]
    pages = [(n + P - 1) // P for n in lens]
    num_pages = sum(pages) + 64
    pt = scatter_pages(pages, num_pages, seed)
    past = [n - 1 for n in lens]
    kp, vp = fill_gqa_pools(past, pt, num_pages, Hkv, P, D, seed)
    q = orc.fill_normal((B, 1, Hq, D), seed + 11)
    k = orc.fill_normal((B, 1, Hkv, D), seed + 12)
    v = orc.fill_normal((B, 1, Hkv, D), seed + 13)
    inv = orc.default_inv_freq(theta, 64)
    pos = np.array(past, np.int32)
    pool = be.prepare_kv_pool(num_pages, P, Hkv, D)
    pool.k.copy_(dev(be, kp).view(torch.float16))
    pool.v.copy_(dev(be, vp).view(torch.float16))
    want = orc.gqa_paged_attention(orc.qk_norm_rope(q, None, inv, 64, 0, positions=pos),
                                   orc.qk_norm_rope(k, None, inv, 64, 0, positions=pos), v, None, kp, vp, pt, past, P)
    rope = be.prepare_rope_table(inv, 64, 1.0)
    # no host mirrors: the launch is sized by max_len alone, as in a replayed CUDA graph
    q16 = be.rope_append_gqa(dev(be, q, torch.float16), dev(be, k, torch.float16), dev(be, v, torch.float16), rope, pool,
                             be.page_table(pt, past, validate_on_host=False))
    outs = [be.gqa_decode_paged(q16[:, 0].contiguous(), pool, be.page_table(pt, lens, validate_on_host=False),
                                max_len=max(lens), split_chunk=c) for c in chunk]
    be.device_flush()
    # appended V rows are copied, not computed: the pools agree bit for bit (kp / vp now hold the oracle's append)
    assert np.array_equal(pool.v.cpu().numpy().view(np.uint16), vp)
    kd = pool.k.cpu().numpy().view(np.uint16).astype(np.int32)
    assert np.abs(kd - kp.astype(np.int32)).max() <= 1
    return [assert_close(o.cpu().numpy(), want[:, 0], f"decode chunk {c}") for o, c in zip(outs, chunk)]


def test_config3_full_size(be):
    """Batch 32, 48 / 8 heads, contexts U{1024..16384} from the benchmark's own seeded draw, split-KV chunk 512,
    16-token pages scattered through one pool, RoPE theta 5e5 + append of the current token.  Every sequence is
    longer than 2048 keys' worth of one CTA or spans several CTAs of a run (f16_attention_kernels.metal:325-510)."""
    from bench import decode_lens
    lens = decode_lens(0, 32)
    assert lens.min() >= 1024 and lens.max() <= 16384 and (lens > 2048).sum() >= 20
    _decode_case(be, lens, 48, 8, [512], SEED0 + 3)


def test_long_sequence_spans_several_ctas(be):
    """One 5000-key sequence: three CTAs per KV head each stream a run of chunks; partial slots are indexed by
    run * chunks_per_cta + chunk.  Chunk 64 (79 partials) and chunk 512 (10 partials)."""
    _decode_case(be, [5000, 2049, 4096], 48, 8, [64, 512, 2048], SEED0 + 33)


def test_mid_sized_batch_takes_runs_of_two_chunks(be):
    """Ten sequences of up to 9 000 keys: too few for two waves of four-chunk runs, so every CTA streams two 512-key
    chunks (a single long sequence takes one chunk per CTA, the benchmark's batch of 32 four)."""
    rng = np.random.RandomState(SEED0 + 35)
    lens = [int(n) for n in rng.randint(600, 9001, size=10)]
    lens[3] = 9000
    _decode_case(be, lens, 48, 8, [512], SEED0 + 36)


def test_length_beyond_max_len_is_cut_and_reported(be):
    """lens[b] > max_len with no host mirror (what a replayed graph with stale sizes would do): the kernels cut the
    sequence to what the launch was sized for, never touch another sequence's partials, and inf_flush reports it."""
    from inferno_b200 import InfernoError
    D, P, Hq, Hkv = 128, 16, 12, 2
    lens = [300, 900, 200]
    pages = [(n + P - 1) // P for n in lens]
    pt = scatter_pages(pages, sum(pages) + 3, SEED0 + 61)
    pool = be.prepare_kv_pool(sum(pages) + 3, P, Hkv, D)
    g = torch.Generator(device=be.device).manual_seed(SEED0 + 62)
    pool.k.normal_(0, 1, generator=g)
    pool.v.normal_(0, 1, generator=g)
    q = torch.randn((3, Hq, D), generator=g, device=be.device, dtype=torch.float16)
    be.device_flush()
    good = be.gqa_decode_paged(q, pool, be.page_table(pt, lens), max_len=900, split_chunk=64)
    be.device_flush()
    # the same launch sized for 320 keys: sequence 1 does not fit
    bad = be.gqa_decode_paged(q, pool, be.page_table(pt, lens, validate_on_host=False), max_len=320, split_chunk=64)
    with pytest.raises(InfernoError) as e:
        be.device_flush()
    assert "length beyond" in str(e.value)
    good, bad = good.cpu().numpy(), bad.cpu().numpy()
    assert np.all(np.isfinite(bad))
    assert np.array_equal(bad[0], good[0]) and np.array_equal(bad[2], good[2])  # the neighbours are untouched
    # sequence 1 was attended over its first 320 keys only
    cut = be.gqa_decode_paged(q, pool, be.page_table(pt, [300, 320, 200]), max_len=320, split_chunk=64)
    be.device_flush()
    assert np.array_equal(bad[1], cut.cpu().numpy()[1])
    # with the host mirror the same call is refused before any launch
    with pytest.raises(InfernoError) as e:
        be.gqa_decode_paged(q, pool, be.page_table(pt, lens), max_len=320, split_chunk=64)
    assert e.value.kind == "ShapeMismatch"
    be.device_flush()


def test_bad_page_id_is_refused_on_the_device(be):
    """A page id outside the pool, with no host mirror: the kernel reads zeros instead (no address is formed from
    the id) and inf_flush reports it."""
    from inferno_b200 import InfernoError
    D, P, Hq, Hkv = 128, 16, 12, 2
    pool = be.prepare_kv_pool(8, P, Hkv, D)
    q = torch.randn((1, Hq, D), device=be.device, dtype=torch.float16)
    out = be.gqa_decode_paged(q, pool, be.page_table([[0, 1, 99, 3]], [60], validate_on_host=False), max_len=64,
                              split_chunk=64)
    with pytest.raises(InfernoError) as e:
        be.device_flush()
    assert "page id outside" in str(e.value)
    assert np.all(np.isfinite(out.cpu().numpy()))
    be.device_flush()  # the status word was cleared by the failed flush


def test_bounded_wait_gives_up_and_the_context_survives(be):
    """A load that never arrives: the consumers' wait runs out (two seconds), the kernel leaves through its normal
    end, inf_flush names the cause, and the very next call on the same context is correct again."""
    import time
    from inferno_b200 import InfernoError
    D, P, Hq, Hkv = 128, 16, 12, 2
    pool = be.prepare_kv_pool(12, P, Hkv, D)
    g = torch.Generator(device=be.device).manual_seed(SEED0 + 71)
    pool.k.normal_(0, 1, generator=g)
    pool.v.normal_(0, 1, generator=g)
    q = torch.randn((1, Hq, D), generator=g, device=be.device, dtype=torch.float16)
    table = be.page_table(np.arange(12, dtype=np.int32)[None], [180])
    good = be.gqa_decode_paged(q, pool, table, max_len=180, split_chunk=64)
    be.device_flush()
    be._check(be._lib.inf_debug_drop_next_load(be._ctx, 0))  # the first 64-key tile of CTA (0, 0, 0) never lands
    t0 = time.time()
    be.gqa_decode_paged(q, pool, table, max_len=180, split_chunk=64)
    with pytest.raises(InfernoError) as e:
        be.device_flush()
    assert "bounded wait gave up" in str(e.value)
    assert 1.0 < time.time() - t0 < 30.0
    again = be.gqa_decode_paged(q, pool, table, max_len=180, split_chunk=64)
    be.device_flush()
    assert np.array_equal(again.cpu().numpy(), good.cpu().numpy())


def test_rmsnorm_rope_pair_matches_oracle(be):
    """laguna_qk_rms_norm_rope_pair_device on the reference's own test shapes (metal/rope.rs:621-710), tol 3e-5."""
    D, rotary, theta, factor, pos = 128, 64, 500000.0, 1.3465736, 7
    qv = (((np.arange(2 * 3 * D) % 43).astype(np.float32) - 21.0) / 16.0).reshape(1, 2, 3, D)
    kv = (((np.arange(2 * 8 * D) % 59).astype(np.float32) - 29.0) / 24.0).reshape(1, 2, 8, D)
    qw = np.float32(0.75) + (np.arange(D) % 5).astype(np.float32) * np.float32(0.0625)
    kw = np.float32(0.875) + (np.arange(D) % 7).astype(np.float32) * np.float32(0.03125)
    inv = orc.default_inv_freq(theta, rotary)
    table = be.prepare_rope_table(inv, rotary, factor)
    qo, ko = be.laguna_qk_rms_norm_rope_pair_device(dev(be, qv), dev(be, kv), dev(be, qw), dev(be, kw), 1e-6, pos, table)
    assert np.max(np.abs(qo.cpu().numpy() - orc.qk_norm_rope(qv, qw, inv, rotary, pos, 1e-6, factor))) <= 3e-5
    assert np.max(np.abs(ko.cpu().numpy() - orc.qk_norm_rope(kv, kw, inv, rotary, pos, 1e-6, factor))) <= 3e-5
    # the single-tensor form of the same kernel (qk_rms_norm_rope_device, rope_kernels.metal:113)
    one = be.qk_rms_norm_rope_device(dev(be, qv), dev(be, qw), 1e-6, pos, table)
    assert np.array_equal(one.cpu().numpy(), qo.cpu().numpy())
    # sliding-layer convention: rotary 128, theta 1e4
    inv2 = orc.default_inv_freq(10000.0, 128)
    t2 = be.prepare_rope_table(inv2, 128, 1.0)
    qo, ko = be.laguna_qk_rms_norm_rope_pair_device(dev(be, qv), dev(be, kv), dev(be, qw), dev(be, kw), 1e-6, 11, t2)
    assert np.max(np.abs(qo.cpu().numpy() - orc.qk_norm_rope(qv, qw, inv2, 128, 11, 1e-6, 1.0))) <= 3e-5
    assert np.max(np.abs(ko.cpu().numpy() - orc.qk_norm_rope(kv, kw, inv2, 128, 11, 1e-6, 1.0))) <= 3e-5


def test_rope_slice_and_mla_postprocess_match_oracle(be):
    # metal/rope.rs:766-804 shape, tol 1e-5
    T, H, R = 32, 64, 64
    x = (((np.arange(T * H * R) % 251) - 125.0) / 64.0).astype(np.float32).reshape(1, T, H, R)
    got = be.rope_slice_device(dev(be, x), R, 7, 10000.0).cpu().numpy()
    assert np.max(np.abs(got - orc.rope_slice_glm(x, 7, 10000.0))) <= 1e-5
    # MLA post-process + paged append
    B, T, L, R, P = 2, 70, 512, 64, 64
    past = [5, 130]
    pages = [(p + T + P - 1) // P for p in past]
    pt = scatter_pages(pages, sum(pages) + 3, SEED0 + 77)
    xin = orc.fill_normal((B, T, L + R), SEED0 + 78, 1.0, False)
    w = (1.0 + 0.1 * orc.fill_normal((L,), SEED0 + 79, 1.0, False)).astype(np.float32)
    pool = be.prepare_mla_pool(sum(pages) + 3)
    lat, rope = be.mla_kv_postprocess_device(dev(be, xin), dev(be, w), 1e-6, 1.0e7, pool, be.page_table(pt, past))
    be.device_flush()
    rows = pool.rows.cpu().numpy().view(np.uint16)
    for b in range(B):
        lat_o, rope_o = orc.mla_kv_postprocess(xin[b], w, T, L, R, past[b], 1.0e7, 1e-6)
        assert np.max(np.abs(lat[b].cpu().numpy() - lat_o)) <= 2e-5
        assert np.max(np.abs(rope[b].cpu().numpy() - rope_o)) <= 2e-5
        want_bits = np.concatenate([lat_o, rope_o], -1).astype(np.float16).view(np.uint16).astype(np.int32)
        for t in range(T):
            tok = past[b] + t
            got_bits = rows[pt[b, tok // P], tok % P].astype(np.int32)
            assert np.abs(got_bits - want_bits[t]).max() <= 1


def test_host_validation_rejects_before_launch(be):
    from inferno_b200 import InfernoError
    pool = be.prepare_kv_pool(8, 16, 2, 128)
    q = torch.zeros((1, 8, 128), dtype=torch.float16, device=be.device)
    with pytest.raises(InfernoError) as e:
        be.gqa_decode_paged(q, pool, be.page_table([[0, 99]], [20]), max_len=32)
    assert e.value.kind == "Cache"
    with pytest.raises(InfernoError) as e:
        be.gqa_decode_paged(q, pool, be.page_table([[0, 1]], [40]), max_len=64)
    assert e.value.kind == "Cache"
    with pytest.raises(InfernoError) as e:
        be.gqa_decode_paged(q[:, :7].contiguous(), pool, be.page_table([[0, 1]], [20]), max_len=32)
    assert e.value.kind == "ShapeMismatch"
    with pytest.raises(InfernoError) as e:
        be.gqa_decode_paged(q, pool, be.page_table([[0, 1]], [20]), max_len=32, split_chunk=100)
    assert e.value.kind == "Config"
    with pytest.raises(InfernoError):
        be.prepare_rope_table(np.ones(31, np.float32), 64, 1.0)
    with pytest.raises(InfernoError):
        be.prepare_rope_table(np.ones(48, np.float32), 96, 1.0)
    with pytest.raises(InfernoError):
        be.prepare_rope_table(np.ones(32, np.float32), 64, 0.0)
    be.device_flush()  # nothing was launched, the status word is clean
