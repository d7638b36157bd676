"""GPU parity: the expanded-head selected-row attention operators (selected_decode_attention_device,
selected_sequence_attention_device) against the oracle, on the reference's own cases (tolerance 1e-5,
metal/attention.rs:2413-2740) and at DSA sizes."""
import numpy as np
import pytest

from oracle import pyoracle as orc
from tests.test_oracle_pins import selected_attention_cases
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


def dev(be, a, dtype=None):
    if a is None:
        return None
    t = torch.from_numpy(np.ascontiguousarray(a)).to(be.device)
    return t if dtype is None else t.to(dtype)


def run(be, q, sk, sv, ck, cv, inc, kv_dtype=torch.float32):
    if q.shape[2] == 1 and sk is not None:
        return be.selected_decode_attention_device(dev(be, q), dev(be, sk, kv_dtype), dev(be, sv, kv_dtype), dev(be, ck),
                                                   dev(be, cv), inc)
    assert inc
    return be.selected_sequence_attention_device(dev(be, q), dev(be, sk), dev(be, sv), dev(be, ck), dev(be, cv))


def test_reference_cases(be):
    for name, q, sk, sv, ck, cv, inc in selected_attention_cases():
        got = run(be, q, sk, sv, ck, cv, inc)
        be.device_flush()
        assert np.abs(got.cpu().numpy() - orc.selected_attention(q, sk, sv, ck, cv, inc)).max() <= 1e-5, name


@pytest.mark.parametrize("B,H,S,T,D,Dv,f16", [
    (1, 64, 2048, 1, 256, 256, False),   # GLM sparse decode: top-2048 rows, expanded 192+64 keys, 256 values
    (2, 64, 2047, 1, 192, 128, True),    # fp16 selected rows (the f16-KV twin of the kernel), odd count
    (1, 8, 100, 8, 256, 256, False),     # speculative batch of eight rows over a selected past
    (1, 4, 0, 33, 96, 40, False),        # first chunk, no past, dims that are not multiples of 32
    (1, 2, 4088, 8, 64, 64, False),      # the kernel's 4096-key limit
])
def test_sizes_match_oracle(be, B, H, S, T, D, Dv, f16):
    seed = SEED0 + 1900 + S + T
    q = orc.fill_normal((B, H, T, D), seed, 1.0, False)
    sk = orc.fill_normal((B, H, S, D), seed + 1, 1.0, f16) if S else None
    sv = orc.fill_normal((B, H, S, Dv), seed + 2, 1.0, f16) if S else None
    ck = orc.fill_normal((B, H, T, D), seed + 3, 1.0, False)
    cv = orc.fill_normal((B, H, T, Dv), seed + 4, 1.0, False)
    got = run(be, q, sk, sv, ck, cv, True, torch.float16 if f16 else torch.float32)
    be.device_flush()
    want = orc.selected_attention(q, sk, sv, ck, cv, True)
    assert np.abs(got.cpu().numpy() - want).max() <= 2e-5


def test_refusals(be):
    from inferno_b200 import InfernoError
    z = lambda *s: torch.zeros(s, dtype=torch.float32, device=be.device)
    with pytest.raises(InfernoError) as e:   # backend.rs:7864: at least one selected token
        be.selected_decode_attention_device(z(1, 2, 1, 8), z(1, 2, 0, 8), z(1, 2, 0, 8), z(1, 2, 1, 8), z(1, 2, 1, 8), True)
    assert "at least one selected token" in str(e.value)
    # beyond the reference kernel's 4096 keys there is no device path: Ok(None)
    assert be.selected_sequence_attention_device(z(1, 1, 8, 8), z(1, 1, 4090, 8), z(1, 1, 4090, 8), z(1, 1, 8, 8),
                                                 z(1, 1, 8, 8)) is None
    be.device_flush()
