"""GPU parity: absorbed-MLA decode over the paged latent cache (tcgen05 kernel) against the CPU oracle."""
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


def run_case(be, past, T, H, seed, sigma=0.5, out_dtype=torch.float32):
    B = len(past)
    pages = [(n + T + P - 1) // P for n in past]
    num_pages = sum(pages) + 5
    pt = scatter_pages(pages, num_pages, seed)
    pool_np = fill_mla_pool(past, pt, num_pages, P, L + R, seed, sigma)
    q = orc.fill_normal((B, T, H, L + R), seed + 21)
    cur = orc.fill_normal((B, T, L + R), seed + 22, sigma)
    scale = 1.0 / math.sqrt(192.0)
    pool_o = pool_np.copy()
    want = orc.mla_absorbed_paged(q, cur, pool_o, pt, past, P, L, R, scale)
    # CUDA path: the current rows are already in their pages (the append kernel is tested on its own)
    pool = be.prepare_mla_pool(num_pages)
    pool.rows.copy_(dev(be, pool_o).view(torch.float16))
    out = be.mla_decode_absorbed(dev(be, q, torch.float16), pool, be.page_table(pt, past), max_len=max(past) + T,
                                 scale=scale, out_dtype=out_dtype)
    be.device_flush()
    return out.float().cpu().numpy(), want


@pytest.mark.parametrize("ctx", [4096, 32768])
def test_config2_absorbed_mla_decode(be, ctx):
    """batch 1, 64 heads, 576-wide shared row, v dim 512, 64-token pages under a seeded random table."""
    got, want = run_case(be, [ctx - 1], 1, 64, SEED0 + 1 + ctx)
    assert_close(got, want, f"config 2 ctx={ctx}")


@pytest.mark.parametrize("past,T,H", [
    ([0], 1, 64),            # a single cached row: output equals its latent
    ([2], 3, 2),             # the reference test's token/head counts (metal/q2.rs:8214-8226): causal current rows
    ([63, 64, 200], 1, 64),  # page boundaries, ragged batch
    ([1000], 2, 128),        # two 64-head blocks
    ([5000, 130], 4, 16),
])
def test_absorbed_mla_decode_matches_oracle(be, past, T, H):
    got, want = run_case(be, past, T, H, SEED0 + 600 + H + T)
    assert_close(got, want, f"mla decode past={past} T={T} H={H}")


def test_fp16_output_and_single_row_identity(be):
    got, want = run_case(be, [0], 1, 64, SEED0 + 650, out_dtype=torch.float16)
    assert_close(got, want, "fp16 out")


def test_postprocess_append_then_decode(be):
    """mla_kv_postprocess_device feeding the decode kernel: rows are normalised, roped, appended, then attended."""
    B, T, H, past = 1, 2, 64, [100]
    seed = SEED0 + 700
    pages = [(past[0] + T + P - 1) // P]
    pt = scatter_pages(pages, 8, seed)
    pool_np = fill_mla_pool(past, pt, 8, P, L + R, seed)
    x = orc.fill_normal((B, T, L + R), seed + 1, 1.0, False)
    w = (1.0 + 0.1 * orc.fill_normal((L,), seed + 2, 1.0, False)).astype(np.float32)
    q = orc.fill_normal((B, T, H, L + R), seed + 3)
    lat, rope = orc.mla_kv_postprocess(x[0], w, T, L, R, past[0], 1.0e7, 1e-6)
    cur = np.concatenate([lat, rope], -1)[None]
    scale = 1.0 / math.sqrt(192.0)
    want = orc.mla_absorbed_paged(q, cur, pool_np.copy(), pt, past, P, L, R, scale)
    pool = be.prepare_mla_pool(8)
    pool.rows.copy_(dev(be, pool_np).view(torch.float16))
    table = be.page_table(pt, past)
    be.mla_kv_postprocess_device(dev(be, x), dev(be, w), 1e-6, 1.0e7, pool, table)
    out = be.mla_decode_absorbed(dev(be, q, torch.float16), pool, table, max_len=past[0] + T, scale=scale)
    be.device_flush()
    assert_close(out.cpu().numpy(), want, "postprocess + decode")
