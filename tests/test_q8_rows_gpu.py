"""GPU parity, bit-exact: the Q8Row cold-store codec and the thaw of cold MLA rows into the paged pool."""
import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0, scatter_pages

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from inferno_b200 import CudaBackend
    b = CudaBackend(0)
    yield b
    b.device_flush()
    b.close()


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(be.device)


def sample_rows(rows, dim, seed):
    x = orc.fill_normal((rows, dim), seed, 1.0, False)
    x[0] = 0.0                       # an all-zero row: scale 1.0
    x[1, :] = np.float32(1e-30)      # a tiny row
    x[2, 0] = np.float32(127.0)      # scale exactly 1: values ending in .5 round away from zero
    x[2, 1:9] = np.array([0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5], np.float32)
    return x


@pytest.mark.parametrize("rows,dim", [(300, 512), (7, 64), (5, 33)])
def test_encode_and_decode_are_bit_exact(be, rows, dim):
    x = sample_rows(rows, dim, SEED0 + 1300 + dim)
    want = orc.q8_rows_encode(x)
    got = be.q8_rows_encode(dev(be, x))
    be.device_flush()
    assert np.array_equal(got.cpu().numpy(), want)
    back = be.q8_rows_decode(got, dim)
    be.device_flush()
    assert np.array_equal(back.cpu().numpy().view(np.uint32), orc.q8_rows_decode(want, dim).view(np.uint32))


def test_thaw_into_pages_is_bit_exact(be):
    L, R, P, B, T, first = 512, 64, 64, 2, 150, 37
    seed = SEED0 + 1350
    pages = [(first + T + P - 1) // P] * B
    pt = scatter_pages(pages, sum(pages) + 2, seed)
    lat = orc.fill_normal((B * T, L), seed + 1, 0.5, False)
    rope = orc.fill_normal((B * T, R), seed + 2, 0.5, False)
    lp, rp = orc.q8_rows_encode(lat), orc.q8_rows_encode(rope)
    pool = be.prepare_mla_pool(sum(pages) + 2)
    before = pool.rows.clone()
    table = be.page_table(pt, [0] * B)
    be.mla_pool_thaw_q8_rows(dev(be, lp), dev(be, rp), pool, table, first, T)
    be.device_flush()
    got = pool.rows.cpu().numpy().view(np.uint16).reshape(-1, P, L + R)
    want = before.cpu().numpy().view(np.uint16).reshape(-1, P, L + R).copy()
    dl = orc.q8_rows_decode(lp, L).astype(np.float16).view(np.uint16).reshape(B, T, L)
    dr = orc.q8_rows_decode(rp, R).astype(np.float16).view(np.uint16).reshape(B, T, R)
    for b in range(B):
        for t in range(T):
            pos = first + t
            want[pt[b, pos // P], pos % P, :L] = dl[b, t]
            want[pt[b, pos // P], pos % P, L:] = dr[b, t]
    assert np.array_equal(got, want)
