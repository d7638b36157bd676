"""GPU parity: sliding-window decode and prefill after the pages below the window went back to the pool
(inf_paged_index_trim) and were overwritten: the kernels must not read, or complain about, a page slot that
lies wholly below the window.  Reference ring: crates/backend/src/metal/f16_attention.rs:120-210."""
import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0, assert_close, fill_gqa_pools

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


def build(be, past, T, W, Hq, Hkv, seed):
    """A sequence of `past` cached rows managed by the page index, trimmed for a query chunk of T rows."""
    from inferno_b200.paged import PagedIndex
    D, P = 128, 16
    num_pages = (past + T) // P + 12
    idx = PagedIndex(num_pages, P, 1, 512)
    if past:
        idx.append(0, past)
    pages, _ = idx.arrays()
    kp, vp = fill_gqa_pools([past], pages[:1].copy(), num_pages, Hkv, P, D, seed)
    released = idx.trim(0, max(0, past + 1 - W))
    assert released == max(0, (past + 1 - W) // P)
    idx.append(0, T)                      # the chunk's own rows may land in pages that were just released
    pages, _ = idx.arrays()
    pt = pages[:1].copy()
    # what the oracle sees: the same rows, but the released pages hold garbage now (they belong to someone else)
    kp_o, vp_o = kp.copy(), vp.copy()
    live = set(int(x) for x in pt[0] if x >= 0)
    for page in range(num_pages):
        if page not in live:
            kp[page] = 0x7bff
            vp[page] = 0xfbff            # +-65504: any read of a released page wrecks the result
    pt_o = pt.copy()
    # the oracle never touches rows below the window either, so -1 entries are never dereferenced; give it a valid id
    pt_o[pt_o < 0] = 0
    q = orc.fill_normal((1, T, Hq, D), seed + 11)
    k = orc.fill_normal((1, T, Hkv, D), seed + 12)
    v = orc.fill_normal((1, T, Hkv, D), seed + 13)
    want = orc.gqa_paged_attention(q, k, v, None, kp_o, vp_o, pt_o, [past], P, sliding_window=W)
    pool = be.prepare_kv_pool(num_pages, P, Hkv, D)
    pool.k.copy_(dev(be, kp).view(torch.float16))
    pool.v.copy_(dev(be, vp).view(torch.float16))
    idx.close()
    return pool, pt, q, k, v, want


@pytest.mark.parametrize("past,W", [(2000, 512), (700, 512), (1030, 64), (300, 512)])
def test_decode_after_trim(be, past, W):
    Hq, Hkv = 48, 8
    pool, pt, q, k, v, want = build(be, past, 1, W, Hq, Hkv, SEED0 + 1700 + past)
    table_past, table_full = be.page_table(pt, [past]), be.page_table(pt, [past + 1])   # host mirrors on: -1 slots below the window pass
    q16 = be.rope_append_gqa(dev(be, q, torch.float16), dev(be, k, torch.float16), dev(be, v, torch.float16), None, pool,
                             table_past)
    out = be.gqa_decode_paged(q16[:, 0].contiguous(), pool, table_full, max_len=past + 1, split_chunk=128,
                              sliding_window=W)
    be.device_flush()                      # no status bit: nothing below the window was resolved
    assert_close(out.cpu().numpy(), want[:, 0], f"decode after trim past={past} W={W}")


@pytest.mark.parametrize("past,T,W", [(1500, 200, 512), (600, 130, 512), (0, 700, 512)])
def test_prefill_chunk_after_trim(be, past, T, W):
    Hq, Hkv = 12, 2
    pool, pt, q, k, v, want = build(be, past, T, W, Hq, Hkv, SEED0 + 1800 + past)
    table = be.page_table(pt, [past])
    q16 = be.rope_append_gqa(dev(be, q, torch.float16), dev(be, k, torch.float16), dev(be, v, torch.float16), None, pool,
                             table)
    out = be.gqa_prefill_paged(q16, pool, table, sliding_window=W, out_dtype=torch.float32)
    be.device_flush()
    assert_close(out.cpu().numpy(), want, f"prefill after trim past={past} T={T} W={W}")
