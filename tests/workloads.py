"""Seeded synthetic workloads shared by the GPU parity tests.

Values come from the oracle's counter-based generator (splitmix64 -> Box-Muller, rounded to
fp16), page tables from its Fisher-Yates permutation, so the oracle and the CUDA path see the
same bits.  Shapes follow the benchmark configurations.
"""
import numpy as np

from oracle import pyoracle as orc

SEED0 = 0x1FE2A0

TOL_ABS, TOL_REL = 2e-3, 1e-2  # the stated fp16-output tolerance: max-abs 2e-3 / rel 1e-2


def assert_close(got, want, what=""):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.all(np.isfinite(got)), f"{what}: non-finite values"
    err = np.abs(got - want)
    bad = err > (TOL_ABS + TOL_REL * np.abs(want))
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} outside max-abs {TOL_ABS} / rel {TOL_REL}; "
                           f"worst abs err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}")
    return float(err.max())


def scatter_pages(batch_pages, num_pages, seed):
    """Page table [batch, max_pages] whose used entries are a seeded random scatter of the pool."""
    total = int(sum(batch_pages))
    assert total <= num_pages
    perm = orc.permutation(num_pages, seed)
    max_pages = int(max(batch_pages))
    table = np.full((len(batch_pages), max_pages), -1, np.int32)
    o = 0
    for b, n in enumerate(batch_pages):
        table[b, :n] = perm[o:o + n]
        o += n
    return table


def fill_gqa_pools(lens, page_table, num_pages, kv_heads, page_size, head_dim, seed, sigma=1.0):
    """K/V pools (uint16 bit patterns) holding `lens[b]` cached rows per sequence, N(0, sigma) fp16."""
    kp = np.zeros((num_pages, kv_heads, page_size, head_dim), np.uint16)
    vp = np.zeros_like(kp)
    for b, n in enumerate(lens):
        if n == 0:
            continue
        k = orc.fill_normal((n, kv_heads, head_dim), seed + 1000 * b + 1, sigma).astype(np.float16).view(np.uint16)
        v = orc.fill_normal((n, kv_heads, head_dim), seed + 1000 * b + 2, sigma).astype(np.float16).view(np.uint16)
        for s in range((n + page_size - 1) // page_size):
            t0, t1 = s * page_size, min(n, (s + 1) * page_size)
            page = page_table[b, s]
            kp[page, :, :t1 - t0] = np.transpose(k[t0:t1], (1, 0, 2))
            vp[page, :, :t1 - t0] = np.transpose(v[t0:t1], (1, 0, 2))
    return kp, vp


def fill_mla_pool(lens, page_table, num_pages, page_size, width, seed, sigma=0.5):
    pool = np.zeros((num_pages, page_size, width), np.uint16)
    for b, n in enumerate(lens):
        if n == 0:
            continue
        rows = orc.fill_normal((n, width), seed + 1000 * b + 7, sigma).astype(np.float16).view(np.uint16)
        for s in range((n + page_size - 1) // page_size):
            t0, t1 = s * page_size, min(n, (s + 1) * page_size)
            pool[page_table[b, s], :t1 - t0] = rows[t0:t1]
    return pool


def collect_ranks(procs, queue, timeout):
    """Start `procs`, take one (rank, ok, detail) tuple per process from `queue`, and never leave a rank behind:
    whatever happens (a rank that raised, one that blocks in a collective, a timeout here) every process still
    alive at the end is terminated, then killed."""
    import queue as queue_mod
    results = []
    try:
        for p in procs:
            p.start()
        for _ in procs:
            try:
                r = queue.get(timeout=timeout)
            except queue_mod.Empty:
                raise AssertionError(f"a rank did not report within {timeout} s; got {results}")
            results.append(r)
            if not r[1]:
                raise AssertionError(f"rank {r[0]} failed: {r[2]}")
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0, f"rank process exited with {p.exitcode}"
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    return results
