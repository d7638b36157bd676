"""GPU parity: absorbed-MLA decode over selected rows (the attention step of DSA sparse decode with the gather
fused into the kernel) against the oracle run on the gathered rows."""
import math

import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0, assert_close, fill_mla_pool, scatter_pages

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

L, R, P = 512, 64, 64


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


def gather_rows(pool, pt, b, ids):
    """fp16 bit patterns of the logical rows `ids` of sequence b."""
    return np.stack([pool[pt[b, i // P], i % P] for i in ids])


def oracle_selected(q, pool, pt, sel, scale):
    """The reference attends to a compact copy of the selected rows (crates/model/src/attention.rs:2843-2960):
    rows 0..n-2 of the list become a compact paged cache, the last listed row plays the current token."""
    B, _, H, _ = q.shape
    out = np.empty((B, 1, H, L), np.float32)
    for b in range(B):
        rows = gather_rows(pool, pt, b, sel[b])
        n = len(rows)
        pages = (n + P - 1) // P
        compact = np.zeros((pages, P, L + R), np.uint16)
        compact.reshape(-1, L + R)[:n - 1] = rows[:n - 1]
        cur = rows[n - 1:].view(np.float16).astype(np.float32).reshape(1, 1, L + R)
        table = np.arange(pages, dtype=np.int32)[None]
        out[b] = orc.mla_absorbed_paged(q[b:b + 1], cur, compact, table, [n - 1], P, L, R, scale)[0]
    return out


def run_case(be, lens, counts, H, seed, order="sorted"):
    B = len(lens)
    pages = [(n + P - 1) // P for n in lens]
    num_pages = sum(pages) + 4
    pt = scatter_pages(pages, num_pages, seed)
    pool_np = fill_mla_pool(lens, pt, num_pages, P, L + R, seed)
    q = orc.fill_normal((B, 1, H, L + R), seed + 41)
    stride = max(counts)
    sel = np.full((B, stride), -7, np.int32)  # entries past the count are never read
    sel_lists = []
    for b in range(B):
        rs = np.random.RandomState(seed + 50 + b)
        ids = rs.permutation(lens[b] - 1)[:counts[b] - 1]
        ids = np.sort(ids) if order == "sorted" else ids
        ids = np.concatenate([ids, [lens[b] - 1]]).astype(np.int32)  # the newest row is always kept
        sel[b, :counts[b]] = ids
        sel_lists.append(ids)
    scale = 1.0 / math.sqrt(192.0)
    want = oracle_selected(q, pool_np, pt, sel_lists, scale)
    pool = be.prepare_mla_pool(num_pages)
    pool.rows.copy_(dev(be, pool_np).view(torch.float16))
    table = be.page_table(pt, [n - 1 for n in lens])  # lens = rows cached before the current token's row
    got = be.mla_decode_absorbed_selected(dev(be, q, torch.float16), pool, table, dev(be, sel),
                                          dev(be, np.array(counts, np.int32)), scale)
    be.device_flush()
    return got.cpu().numpy(), want


@pytest.mark.parametrize("lens,counts,H,order", [
    ([32768], [2048], 64, "sorted"),          # GLM long-context decode: top-2048 of 32 768 rows, 64 heads
    ([4096], [2048], 64, "shuffled"),         # any order gives the same softmax
    ([300, 70, 5000], [65, 64, 1], 64, "sorted"),  # ragged batch: 65 rows (two groups), exactly one group, one row
    ([1000], [63], 3, "sorted"),              # fewer heads than one block
])
def test_selected_rows_match_oracle(be, lens, counts, H, order):
    got, want = run_case(be, lens, counts, H, SEED0 + 950 + H + len(lens), order)
    assert_close(got, want, f"mla selected lens={lens} counts={counts}")


def test_selecting_every_row_equals_the_contiguous_kernel(be):
    """Listing all visible rows must reproduce inf_mla_decode_absorbed bit for bit in the weights' inputs."""
    n, H = 777, 64
    seed = SEED0 + 990
    pt = scatter_pages([(n + P - 1) // P], 20, seed)
    pool_np = fill_mla_pool([n], pt, 20, P, L + R, seed)
    q = dev(be, orc.fill_normal((1, 1, H, L + R), seed + 1), torch.float16)
    pool = be.prepare_mla_pool(20)
    pool.rows.copy_(dev(be, pool_np).view(torch.float16))
    table = be.page_table(pt, [n - 1])
    scale = 1.0 / math.sqrt(192.0)
    full = be.mla_decode_absorbed(q, pool, table, max_len=n, scale=scale)
    sel = dev(be, np.arange(n, dtype=np.int32)[None])
    got = be.mla_decode_absorbed_selected(q, pool, table, sel, dev(be, np.array([n], np.int32)), scale)
    be.device_flush()
    assert_close(got.cpu().numpy(), full.cpu().numpy(), "selected == contiguous")


def test_row_outside_the_sequence_is_reported(be):
    from inferno_b200 import InfernoError
    n = 100
    pt = scatter_pages([2], 6, SEED0 + 995)
    pool = be.prepare_mla_pool(6)
    table = be.page_table(pt, [n - 1])
    q = torch.zeros((1, 1, 64, L + R), dtype=torch.float16, device=be.device)
    sel = dev(be, np.array([[0, 5, n]], np.int32))  # row n is not visible yet
    be.mla_decode_absorbed_selected(q, pool, table, sel, dev(be, np.array([3], np.int32)), 0.07)
    with pytest.raises(InfernoError):
        be.device_flush()


def test_count_beyond_the_list_and_empty_list(be):
    """counts[b] > selected_stride is cut to the stride and reported (the kernel never reads past a sequence's row of
    the list); counts[b] == 0 gives a zero output row instead of a division by zero in the merge."""
    from inferno_b200 import InfernoError
    n, H = 500, 64
    seed = SEED0 + 996
    pt = scatter_pages([8, 8], 20, seed)
    pool_np = fill_mla_pool([n, n], pt, 20, P, L + R, seed)
    pool = be.prepare_mla_pool(20)
    pool.rows.copy_(dev(be, pool_np).view(torch.float16))
    table = be.page_table(pt, [n - 1, n - 1])
    q = dev(be, orc.fill_normal((2, 1, H, L + R), seed + 1), torch.float16)
    ids = np.sort(np.random.RandomState(seed).permutation(n)[:70]).astype(np.int32)
    sel = dev(be, np.stack([ids, ids]))
    scale = 1.0 / math.sqrt(192.0)
    want = be.mla_decode_absorbed_selected(q, pool, table, sel, dev(be, np.array([70, 70], np.int32)), scale)
    be.device_flush()
    got = be.mla_decode_absorbed_selected(q, pool, table, sel, dev(be, np.array([0, 9999], np.int32)), scale)
    with pytest.raises(InfernoError) as e:
        be.device_flush()
    assert "length beyond" in str(e.value)
    got, want = got.cpu().numpy(), want.cpu().numpy()
    assert np.all(got[0] == 0.0)
    assert np.array_equal(got[1], want[1])
    be.device_flush()
