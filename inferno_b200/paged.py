"""Host-side page bookkeeping: Python face of the inf_paged_index_* entry points.

Mirrors the addressing part of the reference's PagedKvCache (crates/cache/src/paged.rs): logical token ->
(physical page, offset), append for prefill and decode, page statistics -- for many sequences over one
shared pool -- plus cheap checkpoints.  Needs no GPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L
from .lib import InfernoError


class PagedIndex:
    def __init__(self, num_pages: int, page_size: int, max_seqs: int, max_pages_per_seq: int):
        self._lib = L.load()
        h = C.c_void_p()
        rc = self._lib.inf_paged_index_create(num_pages, page_size, max_seqs, max_pages_per_seq, C.byref(h))
        if rc != L.INF_OK:
            raise InfernoError(rc, "page index sizes must be positive")
        self._h = h
        self.num_pages, self.page_size, self.max_seqs, self.max_pages = num_pages, page_size, max_seqs, max_pages_per_seq

    def close(self):
        if getattr(self, "_h", None):
            self._lib.inf_paged_index_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != L.INF_OK:
            raise InfernoError(rc, self._lib.inf_paged_index_last_error(self._h).decode())

    def append(self, seq: int, tokens: int):
        """Reserve `tokens` more logical slots; returns (start_position, pages newly allocated)."""
        start, fresh = C.c_int32(), C.c_int32()
        self._check(self._lib.inf_paged_index_append(self._h, seq, tokens, C.byref(start), C.byref(fresh)))
        return start.value, fresh.value

    def token_location(self, seq: int, token: int):
        page, off = C.c_int32(), C.c_int32()
        self._check(self._lib.inf_paged_index_locate(self._h, seq, token, C.byref(page), C.byref(off)))
        return page.value, off.value

    def cached_tokens(self, seq: int) -> int:
        return self._lib.inf_paged_index_len(self._h, seq)

    def page_count(self, seq: int) -> int:
        return self._lib.inf_paged_index_page_count(self._h, seq)

    def free_pages(self) -> int:
        return self._lib.inf_paged_index_free_pages(self._h)

    def page_stats(self, seq: int):
        """[(physical_page_id, start_token, token_count, free_slots)] like PagedKvCache::page_stats."""
        n, P = self.cached_tokens(seq), self.page_size
        pages, _ = self.arrays()
        return [(int(pages[seq, i]), i * P, min(P, n - i * P), P - min(P, n - i * P))
                for i in range((n + P - 1) // P) if pages[seq, i] >= 0]

    def release(self, seq: int):
        self._check(self._lib.inf_paged_index_release(self._h, seq))

    def trim(self, seq: int, first_visible: int) -> int:
        """Return the pages wholly below `first_visible` (the lowest row a future query can see under the sliding
        window) to the pool; logical positions stay.  Returns the number of pages released."""
        n = C.c_int32()
        self._check(self._lib.inf_paged_index_trim(self._h, seq, first_visible, C.byref(n)))
        return n.value

    def checkpoint(self, seq: int):
        self._check(self._lib.inf_paged_index_checkpoint(self._h, seq))

    def restore(self, seq: int):
        self._check(self._lib.inf_paged_index_restore(self._h, seq))

    def arrays(self):
        """(pages int32 [max_seqs, max_pages], lens int32 [max_seqs]) as numpy views of the index's own storage."""
        pp, lp = C.c_void_p(), C.c_void_p()
        ms, mp = C.c_int32(), C.c_int32()
        self._check(self._lib.inf_paged_index_arrays(self._h, C.byref(pp), C.byref(lp), C.byref(ms), C.byref(mp)))
        pages = np.ctypeslib.as_array(C.cast(pp, C.POINTER(C.c_int32)), shape=(ms.value, mp.value))
        lens = np.ctypeslib.as_array(C.cast(lp, C.POINTER(C.c_int32)), shape=(ms.value,))
        return pages, lens
