"""GPU parity, bit-exact: the FP8 E4M3FN KV codec and the dequantisation of FP8 pages into the fp16 pool."""
import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0

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


def test_decode_of_every_byte(be):
    bits = np.arange(256, dtype=np.uint8)
    got = be.fp8_e4m3fn_decode(dev(be, bits), 1.0)
    be.device_flush()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), orc.fp8_e4m3fn_decode(bits).view(np.uint32))


def test_encode_is_bit_exact_incl_ties_saturation_and_subnormals(be):
    vals = [0.0, -0.0, np.nan, 448.0, 449.0, 1e9, -1e9, 464.0, 2.0 ** -6, 2.0 ** -7, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10,
            1.0625, 1.1875, 1.9375, 1.96875, 0.0146484375, 0.01513671875, -0.3, 17.0, 18.0, 19.0, 1e-30, np.inf, -np.inf]
    x = np.concatenate([np.array(vals, np.float32), orc.fill_normal((20000,), SEED0 + 1400, 3.0, False),
                        (orc.fill_normal((5000,), SEED0 + 1401, 1.0, False) * np.float32(1e-2))])
    # every representable value and every midpoint between neighbours (the ties)
    grid = np.sort(orc.fp8_e4m3fn_decode(np.arange(127, dtype=np.uint8)))
    x = np.concatenate([x, grid, (grid[:-1] + grid[1:]) / 2, -grid]).astype(np.float32)
    got = be.fp8_e4m3fn_encode(dev(be, x), 1.0)
    be.device_flush()
    assert np.array_equal(got.cpu().numpy(), orc.fp8_e4m3fn_encode(x))
    # with a scale: encode(x / scale), f32 division
    scale = np.float32(0.37)
    got = be.fp8_e4m3fn_encode(dev(be, x), float(scale))
    be.device_flush()
    assert np.array_equal(got.cpu().numpy(), orc.fp8_e4m3fn_encode((x / scale).astype(np.float32)))


def test_fp8_pages_dequantise_into_the_pool(be):
    num_pages, P, Hkv, D = 11, 16, 8, 128
    rs = np.random.RandomState(SEED0 % 65536 + 77)
    k8 = rs.randint(0, 256, (num_pages, Hkv, P, D)).astype(np.uint8)
    v8 = rs.randint(0, 256, (num_pages, Hkv, P, D)).astype(np.uint8)
    ks, vs = np.float32(0.021), np.float32(1.7)
    pool = be.prepare_kv_pool(num_pages, P, Hkv, D)
    be.kv_pool_from_fp8(dev(be, k8), dev(be, v8), float(ks), float(vs), pool)
    be.device_flush()
    want_k = (orc.fp8_e4m3fn_decode(k8) * ks).astype(np.float32).astype(np.float16)
    want_v = (orc.fp8_e4m3fn_decode(v8) * vs).astype(np.float32).astype(np.float16)
    assert np.array_equal(pool.k.cpu().numpy().view(np.uint16).reshape(want_k.shape), want_k.view(np.uint16))
    assert np.array_equal(pool.v.cpu().numpy().view(np.uint16).reshape(want_v.shape), want_v.view(np.uint16))
