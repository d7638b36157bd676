"""GPU parity: the DSA indexer (index scores, top-k selection) and the whole sparse decode step
scores -> top-k -> absorbed MLA over the selected rows."""
import math

import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.workloads import SEED0, assert_close, fill_mla_pool, scatter_pages

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


@pytest.mark.parametrize("B,past,H,D", [(1, 32767, 32, 128), (3, 100, 4, 64), (2, 0, 8, 128), (1, 63, 32, 128)])
def test_dsa_scores_match_oracle(be, B, past, H, D):
    seed = SEED0 + 1100 + past
    q = orc.fill_normal((B, H, D), seed, 1.0, False)
    w = orc.fill_normal((B, H), seed + 1, 0.3, False)
    pk = orc.fill_normal((B, past, D), seed + 2, 1.0, False) if past else np.zeros((B, 0, D), np.float32)
    ck = orc.fill_normal((B, D), seed + 3, 1.0, False)
    got = be.dsa_scores(dev(be, q), dev(be, w), dev(be, pk), dev(be, ck))
    be.device_flush()
    want = orc.dsa_scores(q, w, pk, ck)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=2e-4, atol=2e-4)
    # against exact arithmetic the kernel must be as good as an fp32 sum (the tensor-core form splits every input
    # into two tf32 terms; a plain tf32 product would miss this bound by two orders of magnitude)
    keys = np.concatenate([pk, ck[:, None, :]], axis=1).astype(np.float64)
    dots = np.einsum("bhd,btd->bth", q.astype(np.float64), keys) / math.sqrt(D)
    exact = np.einsum("bth,bh->bt", np.maximum(dots, 0.0), w.astype(np.float64))
    np.testing.assert_allclose(got.cpu().numpy(), exact, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("B,n,k", [(1, 32768, 2048), (2, 5000, 2048), (1, 100, 2048), (3, 2048, 2048), (1, 4097, 7), (1, 1, 1),
                                   (1, 32769, 2048), (2, 40960, 2048), (1, 45000, 512), (1, 70001, 2048)])
def test_dsa_topk_is_exact(be, B, n, k):
    rs = np.random.RandomState(SEED0 % 65536 + n + k)
    scores = rs.standard_normal((B, n)).astype(np.float32)
    scores[:, ::7] = np.round(scores[:, ::7], 1)  # plenty of exact ties, decided by the lower id
    if n > 10:
        scores[0, 3] = scores[0, 9] = scores[0].max() + 1.0  # a tie at the very top
        scores[:, n // 2] = -0.0
        scores[:, n // 2 + 1] = 0.0
    got = be.dsa_topk(dev(be, scores), k)
    be.device_flush()
    want = orc.dsa_topk(scores, k)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want)


def test_topk_ties_taken_across_rounds_of_the_collection_sweep(be):
    # 100 zeros among the first 32768 tokens (all else -1), zeros after: the 2048 best are the zeros with the lowest ids,
    # 100 from the first round of the sweep and 1948 from the second, the last thread's ties taken in part
    n = 36000
    scores = np.full((1, n), -1.0, np.float32)
    scores[0, 5:32768:331][:100] = 0.0
    scores[0, 32768:] = 0.0
    got = be.dsa_topk(dev(be, scores), 2048)
    be.device_flush()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), orc.dsa_topk(scores, 2048))
    # fewer zeros than k: the threshold falls on -1 and the lowest-id -1 entries fill up
    scores[0, 33000:] = -1.0
    got = be.dsa_topk(dev(be, scores), 2048)
    be.device_flush()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), orc.dsa_topk(scores, 2048))


def test_topk_with_all_equal_scores_takes_the_first_ids(be):
    scores = np.zeros((1, 5000), np.float32)
    got = be.dsa_topk(dev(be, scores), 2048)
    be.device_flush()
    assert np.array_equal(got.cpu().numpy()[0], np.arange(2048, dtype=np.int32))


def test_sparse_decode_step_end_to_end(be):
    """scores -> top-k -> attention over the selected rows, each stage checked against the oracle fed with the
    GPU's own previous stage (so rounding in one stage cannot flip a near-tie in the next)."""
    L, R, P, H = 512, 64, 64, 64
    n, k, Hi, Di = 6000, 2048, 32, 128
    seed = SEED0 + 1200
    q_idx = orc.fill_normal((1, Hi, Di), seed, 1.0, False)
    w_idx = np.abs(orc.fill_normal((1, Hi), seed + 1, 0.3, False))
    keys = orc.fill_normal((1, n, Di), seed + 2, 1.0, False)
    scores = be.dsa_scores(dev(be, q_idx), dev(be, w_idx), dev(be, keys[:, :n - 1]), dev(be, keys[:, n - 1]))
    ids = be.dsa_topk(scores, k)
    be.device_flush()
    assert np.array_equal(ids.cpu().numpy().view(np.uint32), orc.dsa_topk(scores.cpu().numpy(), k))

    pages = [(n + P - 1) // P]
    pt = scatter_pages(pages, pages[0] + 3, seed)
    pool_np = fill_mla_pool([n], pt, pages[0] + 3, P, L + R, seed)
    q = orc.fill_normal((1, 1, H, L + R), seed + 5)
    pool = be.prepare_mla_pool(pages[0] + 3)
    pool.rows.copy_(dev(be, pool_np).view(torch.float16))
    table = be.page_table(pt, [n - 1])
    scale = 1.0 / math.sqrt(192.0)
    counts = torch.tensor([k], dtype=torch.int32, device=be.device)
    got = be.mla_decode_absorbed_selected(dev(be, q).to(torch.float16), pool, table, ids, counts, scale)
    be.device_flush()
    from tests.test_mla_selected_gpu import oracle_selected
    want = oracle_selected(q, pool_np, pt, [ids.cpu().numpy()[0]], scale)
    assert_close(got.cpu().numpy(), want, "sparse decode step")


def test_index_key_layer_norm_and_rope(be):
    B, T, D, rope, pos, theta = 2, 5, 128, 64, 1000, 1.0e4
    seed = SEED0 + 1300
    raw = orc.fill_normal((B, T, D), seed, 2.0, False) + np.float32(0.3)
    wt = orc.fill_normal((D,), seed + 1, 1.0, False)
    bs = orc.fill_normal((D,), seed + 2, 0.1, False)
    got = be.dsa_index_key_device(dev(be, raw), dev(be, wt), dev(be, bs), rope, pos, theta)
    be.device_flush()
    np.testing.assert_allclose(got.cpu().numpy(), orc.dsa_index_key(raw, wt, bs, rope, pos, theta), rtol=2e-5, atol=2e-5)
    # no rotation at all, and a rotation of the whole (short) row
    got = be.dsa_index_key_device(dev(be, raw), dev(be, wt), dev(be, bs), 0, pos, theta)
    be.device_flush()
    np.testing.assert_allclose(got.cpu().numpy(), orc.dsa_index_key(raw, wt, bs, 0, pos, theta), rtol=2e-5, atol=2e-5)
    raw8 = orc.fill_normal((1, 3, 8), seed + 3, 1.0, False)
    got = be.dsa_index_key_device(dev(be, raw8), dev(be, wt[:8].copy()), dev(be, bs[:8].copy()), 8, 7, theta)
    be.device_flush()
    np.testing.assert_allclose(got.cpu().numpy(), orc.dsa_index_key(raw8, wt[:8], bs[:8], 8, 7, theta), rtol=2e-5, atol=2e-5)
    from inferno_b200.lib import InfernoError
    with pytest.raises(InfernoError, match="must be even"):
        be.dsa_index_key_device(dev(be, raw), dev(be, wt), dev(be, bs), 3, pos, theta)


def test_query_rotation_and_head_weights(be):
    B, hidden, H, D, rope, pos, theta = 2, 6144, 32, 128, 64, 4321, 1.0e4
    seed = SEED0 + 1310
    hs = orc.fill_normal((B, hidden), seed, 1.0, False)
    q_raw = orc.fill_normal((B, H * D), seed + 1, 1.0, False)
    proj = orc.fill_normal((hidden, H), seed + 2, 0.02, False)
    q, w = be.dsa_query_weights(dev(be, hs), dev(be, q_raw), dev(be, proj), H, D, rope, pos, theta)
    be.device_flush()
    want_q, want_w = orc.dsa_query_weights(hs, q_raw, proj, H, D, rope, pos, theta)
    np.testing.assert_allclose(q.cpu().numpy(), want_q, rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(w.cpu().numpy(), want_w, rtol=2e-5, atol=2e-5)


def test_decode_topk_chain_reproduces_the_reference_known_answer(be):
    # the reference's own case (two heads of two dims) with every head padded to four dims by zeros, which the score
    # kernels need; the padding adds nothing to a dot product and the ranking does not depend on the 1/sqrt(dim) scale
    hidden = np.array([[[math.sqrt(2.0), 0.0, 0.0, 0.0]]], np.float32)
    q_raw = np.array([[[1.0, 0.0, 0.0, 0.0, 0.0, 1.0, 0.0, 0.0]]], np.float32)
    past = np.array([[[1.0, 0.0, 0.0, 0.0], [0.0, 1.0, 0.0, 0.0], [2.0, 0.0, 0.0, 0.0]]], np.float32)
    cur = np.array([[[0.0, 2.0, 0.0, 0.0]]], np.float32)
    proj = np.array([[1.0, 1.0], [0.0, 0.0], [0.0, 0.0], [0.0, 0.0]], np.float32)
    ids = be.dsa_decode_topk_device(dev(be, hidden), dev(be, q_raw), dev(be, past), dev(be, cur), dev(be, proj), 2, 4, 2, 0,
                                    10000.0, 2)
    be.device_flush()
    assert ids.cpu().numpy().tolist() == [[2, 3]]
    assert orc.dsa_decode_topk(hidden, q_raw, past, cur, proj, 2, 4, 2, 0, 10000.0, 2).tolist() == [[2, 3]]
