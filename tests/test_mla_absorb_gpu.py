"""GPU parity: q8_0_absorbed_mla_device as one call (K_b matvec, absorbed MLA over pages, V_b matvec) and the
per-head Q8_0 matvec on its own, against the CPU oracle composed in the reference's order
(crates/backend/src/metal/device.rs:3537-3584)."""
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


def dev(be, a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(be.device)


def q8_0_weights(heads, out_features, in_features, seed, scale):
    """[heads][out][in] as Q8_0 row blocks: f16 scale (little endian) then 32 signed quants (34 bytes)."""
    nblk = heads * out_features * in_features // 32
    quants = orc.uniform_int(nblk * 32, -127, 127, seed).astype(np.int8).reshape(nblk, 32)
    scales = (scale * (0.5 + orc.uniform_int(nblk, 0, 1000, seed + 1).astype(np.float32) / 1000.0)).astype(np.float16)
    blocks = np.empty((nblk, 34), np.uint8)
    blocks[:, :2] = scales.view(np.uint8).reshape(nblk, 2)
    blocks[:, 2:] = quants.view(np.uint8)
    return blocks.reshape(-1)


def test_packed_q8_heads_closed_form(be):
    """The reference's two-head closed-form case (metal/q2.rs:8173-8209 shapes, row-block layout): constant
    quants per block, f16 scales 1.0 and 2.0."""
    def block(scale_bits, quant):
        return np.concatenate([np.array([scale_bits & 0xFF, scale_bits >> 8], np.uint8),
                               np.full(32, quant, np.int8).view(np.uint8)])
    # heads 2, out 2, in 32
    w = np.concatenate([block(0x3C00, 1), block(0x4000, -2), block(0x4000, 3), block(0x3C00, 1)])
    x = (np.arange(2 * 32, dtype=np.float32).reshape(1, 2, 32) - 20.0) * 0.125
    got = be.q8_0_packed_heads_matvec(dev(be, w), dev(be, x), 2)
    be.device_flush()
    want = np.array([[[x[0, 0].sum(), -4.0 * x[0, 0].sum()], [6.0 * x[0, 1].sum(), x[0, 1].sum()]]], np.float32)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-6, atol=1e-5)
    np.testing.assert_allclose(orc.q8_0_heads_matvec(w, x, 2, 32, 2), want, rtol=1e-6, atol=1e-5)


@pytest.mark.parametrize("rows,heads,fin,fout", [(1, 64, 192, 512), (3, 5, 64, 40), (9, 64, 512, 256),
                                                 (2, 3, 128, 64), (1, 2, 1024, 32), (5, 4, 32, 96)])
def test_packed_q8_heads_matches_oracle(be, rows, heads, fin, fout):
    seed = SEED0 + 800 + rows
    w = q8_0_weights(heads, fout, fin, seed, 0.01)
    x = orc.fill_normal((rows, heads, fin), seed + 5, 1.0, False)
    got = be.q8_0_packed_heads_matvec(dev(be, w), dev(be, x), fout)
    be.device_flush()
    want = orc.q8_0_heads_matvec(w, x, heads, fin, fout)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-4)


def run_absorbed(be, past, T, H, qn, dv, seed, append_inside):
    B = len(past)
    pages = [(n + T + P - 1) // P for n in past]
    num_pages = sum(pages) + 3
    pt = scatter_pages(pages, num_pages, seed)
    pool_np = fill_mla_pool(past, pt, num_pages, P, L + R, seed)
    k_b = q8_0_weights(H, L, qn, seed + 31, 1.0e-3)   # q_latent ~ N(0, 1)
    v_b = q8_0_weights(H, dv, L, seed + 33, 1.0e-3)
    q_no = orc.fill_normal((B, T, H, qn), seed + 35, 1.0, False)
    q_rope = orc.fill_normal((B, T, H, R), seed + 36, 1.0, False)
    cur = orc.fill_normal((B, T, L + R), seed + 37, 0.5)  # fp16-representable, so storing them is exact

    q_lat = orc.q8_0_heads_matvec(k_b, q_no.reshape(B * T, H, qn), H, qn, L).reshape(B, T, H, L)
    q_abs = np.concatenate([q_lat, q_rope], axis=-1)
    pool_o = pool_np.copy()
    ctx = orc.mla_absorbed_paged(q_abs, cur, pool_o, pt, past, P, L, R, 1.0 / math.sqrt(qn + R))
    want = orc.q8_0_heads_matvec(v_b, ctx.reshape(B * T, H, L), H, L, dv).reshape(B, T, H, dv)

    pool = be.prepare_mla_pool(num_pages)
    pool.rows.copy_(dev(be, pool_np if append_inside else pool_o).view(torch.float16))
    table = be.page_table(pt, past)
    lat = dev(be, np.ascontiguousarray(cur[..., :L])) if append_inside else None
    rope = dev(be, np.ascontiguousarray(cur[..., L:])) if append_inside else None
    out = be.q8_0_absorbed_mla_device(dev(be, k_b), dev(be, v_b), dev(be, q_no), dev(be, q_rope), lat, rope, pool,
                                      table, qn + R, dv, max_len=max(past) + T)
    be.device_flush()
    if append_inside:  # the rows the call stored are bit-exact
        assert np.array_equal(pool.rows.cpu().numpy().view(np.uint16).reshape(pool_o.shape), pool_o)
    return out.cpu().numpy(), want


@pytest.mark.parametrize("past,T,H,append_inside", [
    ([4095], 1, 64, True),        # GLM decode shape: 64 heads, q_no_rope 192, value 256, 4096 visible rows
    ([2], 3, 2, True),            # the reference test's token/head counts (metal/q2.rs:8214-8226)
    ([63, 200], 2, 64, False),    # rows already stored by the post-process kernel; ragged batch
    ([0], 1, 7, True),            # a single visible row: out = V_b . that row's latent
])
def test_q8_0_absorbed_mla_matches_oracle(be, past, T, H, append_inside):
    got, want = run_absorbed(be, past, T, H, 192, 256, SEED0 + 900 + H + T, append_inside)
    assert_close(got, want, f"absorbed mla past={past} T={T} H={H}")


def test_q8_0_absorbed_mla_rejects_bad_dims(be):
    from inferno_b200 import InfernoError
    pool = be.prepare_mla_pool(4)
    pt = np.arange(4, dtype=np.int32).reshape(1, 4)
    table = be.page_table(pt, [0])
    z = lambda *s: torch.zeros(s, dtype=torch.float32, device=be.device)
    w = torch.zeros(64, dtype=torch.uint8, device=be.device)
    with pytest.raises(InfernoError):  # qk_head_dim must equal no-RoPE + RoPE (backend.rs:7767)
        be.q8_0_absorbed_mla_device(w, w, z(1, 1, 2, 192), z(1, 1, 2, 64), None, None, pool, table, 192, 256, max_len=1)
    with pytest.raises(InfernoError):  # input width divisible by the Q8_0 block (metal/q2.rs:2673)
        be.q8_0_absorbed_mla_device(w, w, z(1, 1, 2, 100), z(1, 1, 2, 64), None, None, pool, table, 164, 256, max_len=1)
