"""CPU tests: the C ABI exports what the header declares, and the host-side page bookkeeping behaves like
the reference's PagedKvCache (crates/cache/src/paged.rs:498-684)."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "inferno_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(inf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import ctypes
    from inferno_b200 import lib as L
    names = header_functions()
    assert len(names) >= 40
    cdll = ctypes.CDLL(L.LIB_PATH)
    missing = [n for n in names if not hasattr(cdll, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    # and the ctypes table covers the same set, so the Python binding cannot drift from the header
    assert sorted(L.SIGNATURES) == names
    L.load()


def test_context_creation_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import ctypes as C
    from inferno_b200 import lib as L
    h = C.c_void_p()
    assert L.load().inf_ctx_create(0, None, C.byref(h)) == L.INF_E_BACKEND and not h.value
    from inferno_b200 import CudaBackend
    with pytest.raises(RuntimeError):
        CudaBackend(0)


def make(page_size, max_context, seqs=1, pool=None):
    from inferno_b200.paged import PagedIndex
    max_pages = (max_context + page_size - 1) // page_size
    return PagedIndex(pool if pool is not None else max_pages * seqs, page_size, seqs, max_pages)


def test_page_boundaries_map_logical_tokens_to_page_offsets():
    idx = make(4, 16)
    assert idx.append(0, 7) == (0, 2)     # prefill of 7 tokens: pages 0, 1
    assert idx.append(0, 1) == (7, 0)     # decode fills the last slot of page 1
    assert idx.append(0, 1) == (8, 1)     # the next decode opens page 2
    assert idx.cached_tokens(0) == 9 and idx.page_count(0) == 3
    assert idx.token_location(0, 0) == (0, 0)
    assert idx.token_location(0, 3) == (0, 3)
    assert idx.token_location(0, 4) == (1, 0)
    assert idx.token_location(0, 8) == (2, 0)
    stats = idx.page_stats(0)
    assert [(s[2], s[3]) for s in stats] == [(4, 0), (4, 0), (1, 3)]
    assert [s[1] for s in stats] == [0, 4, 8]


def test_decode_appends_into_existing_page_and_allocates_when_full():
    idx = make(4, 8)
    idx.append(0, 3)
    assert idx.append(0, 1) == (3, 0)      # no new page: allocated_pages == 0
    idx2 = make(2, 8)
    idx2.append(0, 2)
    assert idx2.append(0, 1) == (2, 1)     # page full: one new page
    assert idx2.page_count(0) == 2 and idx2.token_location(0, 2) == (1, 0)


def test_token_location_rejects_out_of_range_index():
    from inferno_b200 import InfernoError
    idx = make(2, 8)
    idx.append(0, 1)
    with pytest.raises(InfernoError) as e:
        idx.token_location(0, 1)
    assert "outside cached token count" in str(e.value) and e.value.kind == "Cache"


def test_capacity_pool_exhaustion_release_and_checkpoint():
    from inferno_b200 import InfernoError
    idx = make(4, 16, seqs=3, pool=6)
    idx.append(0, 9)                       # 3 pages
    idx.append(1, 8)                       # 2 pages
    with pytest.raises(InfernoError):
        idx.append(2, 9)                   # needs 3, only 1 free
    with pytest.raises(InfernoError):
        idx.append(0, 8)                   # beyond max_context 16
    pages, lens = idx.arrays()
    assert list(lens) == [9, 8, 0]
    used = [int(p) for p in pages[:2].ravel() if p >= 0]
    assert len(used) == 5 and len(set(used)) == 5 and all(0 <= p < 6 for p in used)
    idx.checkpoint(0)
    idx.append(0, 4)                       # 13 tokens: a 4th page
    assert idx.free_pages() == 0
    idx.restore(0)                         # back to 9 tokens, page given back
    assert idx.cached_tokens(0) == 9 and idx.page_count(0) == 3 and idx.free_pages() == 1
    idx.release(1)
    assert idx.free_pages() == 3 and idx.cached_tokens(1) == 0
    idx.append(2, 9)                       # now it fits


def test_sharding_helpers():
    from inferno_b200.sharding import shard_heads, shard_sequences
    assert shard_heads(48, 8, 1, 0) == (0, 48, 0, 8)
    assert [shard_heads(48, 8, 4, r) for r in range(4)] == [(0, 12, 0, 2), (12, 24, 2, 4), (24, 36, 4, 6), (36, 48, 6, 8)]
    assert shard_heads(64, 64, 8, 7) == (56, 64, 56, 64)
    with pytest.raises(ValueError):
        shard_heads(48, 8, 3, 0)
    cover = [shard_sequences(32, 8, r) for r in range(8)]
    assert cover[0] == (0, 4) and cover[-1] == (28, 32)
    cover = [shard_sequences(10, 4, r) for r in range(4)]
    assert cover == [(0, 3), (3, 6), (6, 8), (8, 10)]


def test_balanced_sequence_order_evens_out_the_keys_per_rank():
    from inferno_b200.sharding import balanced_sequence_order, shard_sequences
    rng = np.random.RandomState(5)
    for world in (1, 2, 4, 8):
        lens = rng.randint(1024, 16385, size=32)
        order = balanced_sequence_order(lens, world)
        assert sorted(order) == list(range(32))          # a permutation
        loads = [int(lens[order[slice(*shard_sequences(32, world, r))]].sum()) for r in range(world)]
        plain = [int(lens[slice(*shard_sequences(32, world, r))].sum()) for r in range(world)]
        assert max(loads) <= max(plain)
        assert max(loads) - min(loads) <= 16384 // 4      # far inside one long sequence
    # ragged block sizes keep their sizes
    order = balanced_sequence_order([5, 1, 9, 7, 3, 8, 2, 6, 4, 10], 4)
    assert sorted(order) == list(range(10)) and len(order) == 10
    assert balanced_sequence_order([], 3) == []


def test_trim_returns_pages_below_the_window_and_keeps_positions():
    """The sliding-window ring on pages: a 512-token window over a growing sequence holds a bounded number of pages
    (the reference's sliding cache is 512 slots, metal/f16_attention.rs:120-210)."""
    from inferno_b200 import InfernoError
    from inferno_b200.paged import PagedIndex
    P, W = 16, 512
    idx = PagedIndex(num_pages=40, page_size=P, max_seqs=2, max_pages_per_seq=256)
    idx.append(0, 600)
    assert idx.page_count(0) == 38 and idx.free_pages() == 2
    released = idx.trim(0, 600 + 1 - W)          # the next query sits at position 600
    assert released == (600 + 1 - W) // P == 5 and idx.free_pages() == 7 and idx.page_count(0) == 33
    pages, lens = idx.arrays()
    assert lens[0] == 600 and (pages[0, :5] == -1).all() and (pages[0, 5:38] >= 0).all()
    assert idx.token_location(0, 599)[1] == 599 % P       # logical positions did not move
    with pytest.raises(InfernoError) as e:
        idx.token_location(0, 10)
    assert "trimmed" in str(e.value)
    # decoding on: the sequence grows to 3000 tokens inside a 40-page pool
    for pos in range(600, 3000):
        idx.append(0, 1)
        idx.trim(0, pos + 2 - W)
        assert idx.page_count(0) <= W // P + 2
    assert idx.cached_tokens(0) == 3000 and idx.trim(0, 0) == 0
    # a checkpoint pins its rows: trimming past it is refused, restoring below the trimmed rows too
    idx.checkpoint(0)
    idx.append(0, 64)
    with pytest.raises(InfernoError) as e:
        idx.trim(0, 3010)
    assert "checkpoint" in str(e.value)
    idx.restore(0)
    assert idx.cached_tokens(0) == 3000
    idx.release(0)
    assert idx.free_pages() == 40 and idx.page_count(0) == 0
    idx.append(0, 5)
    assert idx.token_location(0, 0)[1] == 0
    idx.close()
