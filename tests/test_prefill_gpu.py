"""GPU parity: causal GQA prefill over pages and causal MLA prefill (tcgen05 kernels) against the CPU oracle."""
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


def run_gqa_prefill(be, past, T, Hq, Hkv, window, use_gate, theta=500000.0, rotary=64, seed=SEED0 + 400,
                    out_dtype=None):
    D, P = 128, 16
    B = len(past)
    pages = [(n + T + P - 1) // P for n in past]
    num_pages = sum(pages) + 9
    pt = scatter_pages(pages, num_pages, seed)
    kp, vp = fill_gqa_pools(past, pt, num_pages, Hkv, P, D, seed)
    q = orc.fill_normal((B, T, Hq, D), seed + 11)
    k = orc.fill_normal((B, T, Hkv, D), seed + 12)
    v = orc.fill_normal((B, T, Hkv, D), seed + 13)
    gate = orc.fill_normal((B, T, Hq), seed + 14, 2.0, False) if use_gate else None
    inv = orc.default_inv_freq(theta, rotary)
    pos = np.array(past, np.int32)
    q_r = orc.qk_norm_rope(q, None, inv, rotary, 0, positions=pos)
    k_r = orc.qk_norm_rope(k, None, inv, rotary, 0, positions=pos)
    kp_o, vp_o = kp.copy(), vp.copy()
    want = orc.gqa_paged_attention(q_r, k_r, v, gate, kp_o, vp_o, pt, past, P, sliding_window=window)

    rope = be.prepare_rope_table(inv, rotary, 1.0)
    pool = be.prepare_kv_pool(num_pages, P, Hkv, D)
    pool.k.copy_(dev(be, kp).view(torch.float16))
    pool.v.copy_(dev(be, vp).view(torch.float16))
    table = be.page_table(pt, past)
    q16 = be.rope_append_gqa(dev(be, q, torch.float16), dev(be, k, torch.float16), dev(be, v, torch.float16), rope, pool,
                             table)
    out = be.gqa_prefill_paged(q16, pool, table, sliding_window=window, gate=dev(be, gate) if use_gate else None,
                               out_dtype=out_dtype or torch.float32)
    be.device_flush()
    assert np.array_equal(pool.v.cpu().numpy().view(np.uint16), vp_o)  # appended V pages are bit-exact
    return out.float().cpu().numpy(), want


@pytest.mark.parametrize("past,T,Hq,Hkv,window,use_gate", [
    ([0], 8, 48, 8, 0, True),            # the reference's 8-token prefill shape (metal/f16_attention.rs:792-842)
    ([0], 200, 12, 2, 0, False),         # ragged last query tile
    ([37, 300], 130, 12, 2, 0, True),    # chunked prefill on top of cached tokens, two sequences
    ([0], 300, 8, 8, 100, False),        # sliding window inside the chunk
    ([700], 64, 16, 2, 512, False),      # sliding window reaching into the cache
    ([1], 1, 6, 1, 0, False),            # one row, two keys
])
def test_gqa_prefill_matches_oracle(be, past, T, Hq, Hkv, window, use_gate):
    got, want = run_gqa_prefill(be, past, T, Hq, Hkv, window, use_gate)
    assert_close(got, want, f"gqa prefill past={past} T={T}")


def test_gqa_prefill_config4_full_size(be):
    """2048-token prompt, 48 q / 8 kv heads, theta 5e5, 16-token pages, causal; fp16 output."""
    got, want = run_gqa_prefill(be, [0], 2048, 48, 8, 0, False, out_dtype=torch.float16, seed=SEED0 + 4)
    assert_close(got, want, "config 4")


def test_prefill_then_decode_consistent(be):
    """A row computed by the prefill kernel equals the same row computed by the decode kernel over the cache."""
    D, P, Hq, Hkv, T = 128, 16, 48, 8, 257
    seed = SEED0 + 450
    pt = scatter_pages([(T + P - 1) // P], 40, seed)
    pool = be.prepare_kv_pool(40, P, Hkv, D)
    q = dev(be, orc.fill_normal((1, T, Hq, D), seed + 1), torch.float16)
    k = dev(be, orc.fill_normal((1, T, Hkv, D), seed + 2), torch.float16)
    v = dev(be, orc.fill_normal((1, T, Hkv, D), seed + 3), torch.float16)
    rope = be.prepare_rope_table(orc.default_inv_freq(500000.0, 64), 64, 1.0)
    table = be.page_table(pt, [0])
    q16 = be.rope_append_gqa(q, k, v, rope, pool, table)
    pre = be.gqa_prefill_paged(q16, pool, table, out_dtype=torch.float32)
    dec = be.gqa_decode_paged(q16[:, T - 1].contiguous(), pool, be.page_table(pt, [T]), max_len=T, split_chunk=64)
    be.device_flush()
    assert_close(pre[0, T - 1].cpu().numpy(), dec[0].cpu().numpy(), "prefill row vs decode")


def mla_inputs(T, H, seed, device):
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn((T, H, 192), generator=g, device=device, dtype=torch.float16)
    kn = torch.randn((T, H, 128), generator=g, device=device, dtype=torch.float16)
    kr = torch.randn((T, 64), generator=g, device=device, dtype=torch.float16)
    v = torch.randn((T, H, 128), generator=g, device=device, dtype=torch.float16)
    return q, kn, kr, v


@pytest.mark.parametrize("T,H", [(1, 2), (63, 3), (300, 4), (1000, 2)])
def test_mla_prefill_matches_oracle(be, T, H):
    q, kn, kr, v = mla_inputs(T, H, SEED0 + 500 + T, be.device)
    scale = 1.0 / math.sqrt(192.0)
    out = be.causal_sequence_attention_device(q, kn, kr, v, scale, out_dtype=torch.float32)
    be.device_flush()
    want = orc.causal_mha(q.float().cpu().numpy(), kn.float().cpu().numpy(), kr.float().cpu().numpy(),
                          v.float().cpu().numpy(), scale)
    assert_close(out.cpu().numpy(), want, f"mla prefill T={T}")


def test_mla_prefill_heads_major_layout_and_plain_mha(be):
    """The reference passes [batch, heads, tokens, dim] (backend.rs:8013-8067); strides make that a view."""
    T, H = 200, 3
    q, kn, kr, v = mla_inputs(T, H, SEED0 + 520, be.device)
    scale = 1.0 / math.sqrt(192.0)
    ref = be.causal_sequence_attention_device(q, kn, kr, v, scale, out_dtype=torch.float32)
    qh = q.permute(1, 0, 2).contiguous().permute(1, 0, 2)   # heads-major storage, token-major view
    knh = kn.permute(1, 0, 2).contiguous().permute(1, 0, 2)
    vh = v.permute(1, 0, 2).contiguous().permute(1, 0, 2)
    out = be.causal_sequence_attention_device(qh, knh, kr, vh, scale, out_dtype=torch.float32)
    be.device_flush()
    assert torch.equal(out, ref)
    # no rope tail: plain causal MHA with head_dim 128
    out2 = be.causal_sequence_attention_device(q[..., :128].contiguous(), kn, None, v, 1.0 / math.sqrt(128.0),
                                               out_dtype=torch.float32)
    be.device_flush()
    want = orc.causal_mha(q[..., :128].float().cpu().numpy(), kn.float().cpu().numpy(), None, v.float().cpu().numpy(),
                          1.0 / math.sqrt(128.0))
    assert_close(out2.cpu().numpy(), want, "plain mha")


def test_mla_prefill_config5_sampled_rows(be):
    """32768-token prompt, 64 heads, qk 192, v 128: all rows on the GPU, a seeded sample of rows on the oracle
    (always rows 0, 1, 63, 64, T-1), each against its full causal key range."""
    T, H = 32768, 64
    q, kn, kr, v = mla_inputs(T, H, SEED0 + 5, be.device)
    scale = 1.0 / math.sqrt(192.0)
    out = be.causal_sequence_attention_device(q, kn, kr, v, scale, out_dtype=torch.float16)
    be.device_flush()
    rows = sorted(set([0, 1, 63, 64, T - 1] + list(orc.uniform_int(19, 0, T - 1, SEED0 + 55))))
    idx = torch.tensor(rows, device=be.device)
    want = orc.causal_mha(q.float().cpu().numpy(), kn.float().cpu().numpy(), kr.float().cpu().numpy(),
                          v.float().cpu().numpy(), scale, rows=np.array(rows, np.int32))
    assert_close(out[idx].float().cpu().numpy(), want, "config 5 sampled rows")
    # size-independent property: row 0 attends to one key only, so it equals V[0]
    assert torch.equal(out[0], v[0])
