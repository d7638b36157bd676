"""Two-GPU test of the head-sharded MLA prefill with the NCCL all-gather of the C ABI (inf_comm_*,
inf_allgather_heads): each rank computes its half of the heads with the tcgen05 kernel, the gathered
result must equal the single-GPU result bit for bit.  Skipped on boxes with fewer than two GPUs."""
import math
import os

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, uid_q, res_q):
    import traceback
    try:
        _rank_body(rank, world, uid_q, res_q)
    except Exception:  # report instead of leaving the parent to time out
        res_q.put((rank, False, traceback.format_exc()))


def _rank_body(rank, world, uid_q, res_q):
    import sys
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    from inferno_b200 import CudaBackend
    from inferno_b200.sharding import shard_heads
    torch.cuda.set_device(rank)
    be = CudaBackend(rank)
    if rank == 0:
        uid = be.comm_unique_id()
        for _ in range(world - 1):
            uid_q.put(uid)
    else:
        uid = uid_q.get(timeout=120)
    be.comm_init(uid, rank, world)
    T, H = 384, 8
    g = torch.Generator(device=be.device).manual_seed(1234)
    q = torch.randn((T, H, 192), generator=g, device=be.device, dtype=torch.float16)
    kn = torch.randn((T, H, 128), generator=g, device=be.device, dtype=torch.float16)
    kr = torch.randn((T, 64), generator=g, device=be.device, dtype=torch.float16)
    v = torch.randn((T, H, 128), generator=g, device=be.device, dtype=torch.float16)
    scale = 1.0 / math.sqrt(192.0)
    full = be.causal_sequence_attention_device(q, kn, kr, v, scale)
    qb, qe, kb, ke = shard_heads(H, H, world, rank)
    local = be.causal_sequence_attention_device(q[:, qb:qe].contiguous(), kn[:, kb:ke].contiguous(), kr,
                                                v[:, kb:ke].contiguous(), scale)
    gathered = be.allgather_heads(local)
    be.device_flush()
    res_q.put((rank, bool(torch.equal(gathered, full)), "gathered output differs from the single-GPU result"))
    be.close()


def test_head_sharded_prefill_allgather_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    uid_q, res_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, uid_q, res_q)) for r in range(2)]
    from tests.workloads import collect_ranks
    results = collect_ranks(procs, res_q, timeout=300)
    assert sorted(r[0] for r in results) == [0, 1]
