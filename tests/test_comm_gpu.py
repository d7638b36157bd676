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


def _fused_worker(rank, world, uid_q, inboxes, res_q):
    import traceback
    try:
        _fused_body(rank, world, uid_q, inboxes, res_q)
    except Exception:
        res_q.put((rank, False, traceback.format_exc()))


def _fused_body(rank, world, uid_q, inboxes, res_q):
    """The all-gather fused into the kernels: every rank stores its heads (prefill) or its sequences (decode) into
    its own and, over NVLink, into the peers' copies of the gathered tensor; after the barrier each copy must equal
    the single-GPU result."""
    import sys
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import numpy as np
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
    g = torch.Generator(device=be.device).manual_seed(4321)
    scale = 1.0 / math.sqrt(192.0)
    # ---- dense MLA prefill: gathered [T, H, 128]
    T, H = 300, 8
    q = torch.randn((T, H, 192), generator=g, device=be.device, dtype=torch.float16)
    kn = torch.randn((T, H, 128), generator=g, device=be.device, dtype=torch.float16)
    kr = torch.randn((T, 64), generator=g, device=be.device, dtype=torch.float16)
    v = torch.randn((T, H, 128), generator=g, device=be.device, dtype=torch.float16)
    gathered = torch.zeros((T, H, 128), dtype=torch.float16, device=be.device)
    # ---- paged GQA prefill: gathered [1, T2, Hq, 128]
    T2, Hq, Hkv, P = 200, 12, 4, 16
    q2 = torch.randn((1, T2, Hq, 128), generator=g, device=be.device, dtype=torch.float16)
    k2 = torch.randn((1, T2, Hkv, 128), generator=g, device=be.device, dtype=torch.float16)
    v2 = torch.randn((1, T2, Hkv, 128), generator=g, device=be.device, dtype=torch.float16)
    gathered2 = torch.zeros((1, T2, Hq, 128), dtype=torch.float16, device=be.device)
    # ---- paged GQA decode sharded by sequence: gathered [B3, Hq, 128]
    B3 = 4
    lens3 = np.array([700, 33, 2049, 1200], np.int32)
    q3 = torch.randn((B3, Hq, 128), generator=g, device=be.device, dtype=torch.float16)
    gathered3 = torch.zeros((B3, Hq, 128), dtype=torch.float16, device=be.device)
    torch.cuda.synchronize()
    mine = (be.peer_export(gathered), be.peer_export(gathered2), be.peer_export(gathered3))
    for r in range(world):
        if r != rank:
            inboxes[r].put((rank, mine))
    theirs = dict(inboxes[rank].get(timeout=120) for _ in range(world - 1))
    peers = [be.peer_open(theirs[r][0]) for r in sorted(theirs)]
    peers2 = [be.peer_open(theirs[r][1]) for r in sorted(theirs)]
    peers3 = [be.peer_open(theirs[r][2]) for r in sorted(theirs)]
    assert be.comm_barrier_is_p2p(), "the peers' flag arrays could not be mapped: the barrier fell back to NCCL"
    be.comm_barrier()            # every copy exists and is zero before anybody stores into it
    be.device_flush()

    full = be.causal_sequence_attention_device(q, kn, kr, v, scale)
    qb, qe, kb, ke = shard_heads(H, H, world, rank)
    be.causal_sequence_attention_device(q[:, qb:qe].contiguous(), kn[:, kb:ke].contiguous(), kr, v[:, kb:ke].contiguous(),
                                        scale, out=gathered[:, qb:qe], peers=peers)

    pages = (T2 + P - 1) // P
    table_np = np.arange(pages, dtype=np.int32)[None]
    pool_full = be.prepare_kv_pool(pages, P, Hkv)
    q16 = be.rope_append_gqa(q2, k2, v2, None, pool_full, be.page_table(table_np, [0]))
    full2 = be.gqa_prefill_paged(q16, pool_full, be.page_table(table_np, [0]))
    qb2, qe2, kb2, ke2 = shard_heads(Hq, Hkv, world, rank)
    pool = be.prepare_kv_pool(pages, P, ke2 - kb2)
    q16l = be.rope_append_gqa(q2[:, :, qb2:qe2].contiguous(), k2[:, :, kb2:ke2].contiguous(), v2[:, :, kb2:ke2].contiguous(),
                              None, pool, be.page_table(table_np, [0]))
    be.gqa_prefill_paged(q16l, pool, be.page_table(table_np, [0]), out=gathered2[:, :, qb2:qe2], peers=peers2)

    from inferno_b200.sharding import shard_sequences
    from tests.workloads import scatter_pages
    pages3 = (lens3 + P - 1) // P
    table3 = scatter_pages(list(pages3), int(pages3.sum()) + 5, 99)
    pool3 = be.prepare_kv_pool(int(pages3.sum()) + 5, P, Hkv)
    gk = torch.Generator(device=be.device).manual_seed(77)   # the same cache on every rank
    pool3.k.normal_(0, 1, generator=gk)
    pool3.v.normal_(0, 1, generator=gk)
    full3 = be.gqa_decode_paged(q3, pool3, be.page_table(table3, lens3), int(lens3.max()), 512, out_dtype=torch.float16)
    b0, b1 = shard_sequences(B3, world, rank)
    be.gqa_decode_paged(q3[b0:b1], pool3, be.page_table(table3[b0:b1], lens3[b0:b1]), int(lens3.max()), 512,
                        out=gathered3[b0:b1], peers=peers3)
    be.comm_barrier()
    be.device_flush()
    ok = bool(torch.equal(gathered, full)) and bool(torch.equal(gathered2, full2)) and bool(torch.equal(gathered3, full3))
    be.comm_barrier()            # nobody unmaps a copy a peer's kernel could still be writing
    be.device_flush()
    res_q.put((rank, ok, "a gathered copy differs from the single-GPU result"))
    be.close()


def test_prefill_with_the_gather_fused_into_its_epilogue_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from tests.workloads import collect_ranks
    ctx = mp.get_context("spawn")
    world = 2
    uid_q, res_q = ctx.Queue(), ctx.Queue()
    inboxes = [ctx.Queue() for _ in range(world)]
    procs = [ctx.Process(target=_fused_worker, args=(r, world, uid_q, inboxes, res_q)) for r in range(world)]
    results = collect_ranks(procs, res_q, timeout=300)
    assert sorted(r[0] for r in results) == list(range(world))


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
