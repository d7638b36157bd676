"""The allocation-free decode entry point (inf_gqa_decode_paged_static) against the regular one.

Some callers cannot let the library call cudaMalloc while they decode -- all free HBM already belongs
to their KV pool, or they cannot take the device-wide stall an allocation brings -- so this entry
point keeps its split-KV partials in a fixed array inside the library.  It must return what
inf_gqa_decode_paged returns, call after call, although the array still holds the previous call's
partials.  The file name sorts last on purpose: a failure here cannot hide the other tests.
"""
import numpy as np
import pytest

from tests.workloads import SEED0, TOL_ABS, TOL_REL, scatter_pages

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _case(be, ref_be, lens, Hq, Hkv, chunk, seed, first_call):
    """`be` is a context that has never run a regular decode (its cudaMalloc'ed workspace does not exist), so the
    static entry point cannot be leaning on it; the regular entry point runs on `ref_be`, a second context."""
    D, P = 128, 16
    pages = [(n + P - 1) // P for n in lens]
    num_pages = sum(pages) + 5
    pt = scatter_pages(pages, num_pages, seed)
    pool = be.prepare_kv_pool(num_pages, P, Hkv, D)
    g = torch.Generator(device=be.device).manual_seed(seed)
    pool.k.normal_(0, 1, generator=g)
    pool.v.normal_(0, 1, generator=g)
    q = torch.randn((len(lens), Hq, D), generator=g, device=be.device, dtype=torch.float16)
    table = be.page_table(pt, lens)
    got = torch.full((len(lens), Hq, D), float("nan"), dtype=torch.float32, device=be.device)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(be.device)[0]
    be.gqa_decode_paged_static(q, pool, table, max_len=max(lens), split_chunk=chunk, out=got)
    be.device_flush()
    free_after = torch.cuda.mem_get_info(be.device)[0]
    if not first_call:
        # the very first call of a process may make the driver load the kernels' code; after that a call must leave
        # the device's free memory exactly as it found it
        assert free_after == free_before, f"the static entry point changed free device memory by {free_before - free_after} bytes"
    ref_table = ref_be.page_table(pt, lens)
    want = ref_be.gqa_decode_paged(q, pool, ref_table, max_len=max(lens), split_chunk=chunk)
    ref_be.device_flush()
    want, got = want.cpu().numpy(), got.cpu().numpy()
    assert np.all(np.isfinite(got))
    assert np.all(np.abs(got - want) <= TOL_ABS + TOL_REL * np.abs(want))
    # same kernels, same launch geometry: the two entry points agree to the last bit
    assert np.array_equal(got, want)


def test_static_scratch_decode_matches_regular_entry_point_twice():
    from inferno_b200 import CudaBackend, InfernoError
    be, ref_be = CudaBackend(0), CudaBackend(0)
    try:
        # two calls in a row with different shapes: the second one finds the first one's partials in the array
        _case(be, ref_be, [1500, 64, 2049, 700], 48, 8, 512, SEED0 + 901, first_call=True)
        _case(be, ref_be, [300, 1000], 12, 2, 64, SEED0 + 902, first_call=False)
        _case(be, ref_be, [5000, 33], 48, 8, 512, SEED0 + 903, first_call=False)
        # a request beyond the built-in array is refused with a clear error and nothing is launched
        pool = be.prepare_kv_pool(4, 16, 8, 128)
        q = torch.zeros((64, 48, 128), dtype=torch.float16, device=be.device)
        out = torch.zeros((64, 48, 128), dtype=torch.float32, device=be.device)
        table = be.page_table(np.zeros((64, 4096), np.int32), np.full(64, 16, np.int32), validate_on_host=False)
        with pytest.raises(InfernoError) as e:
            be.gqa_decode_paged_static(q, pool, table, max_len=65536, split_chunk=64, out=out)
        assert e.value.kind == "Config" and "built-in array" in str(e.value)
        be.device_flush()
    finally:
        be.close()
        ref_be.close()
