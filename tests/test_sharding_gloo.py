"""world_size-2 gloo test of the multi-GPU plumbing on CPU: head-sharded attention + all-gather equals the
unsharded result, and sequence sharding covers the batch.  The per-rank attention here is the CPU oracle
(this is a test of the sharding logic, not of the kernels)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out):
    import traceback
    try:
        _rank_body(rank, world, port, q_out)
    except Exception:  # report instead of leaving the parent to time out
        q_out.put((rank, False, traceback.format_exc()))


def _rank_body(rank, world, port, q_out):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from inferno_b200.sharding import allgather_heads, shard_heads, shard_sequences
    from oracle import pyoracle as orc
    T, H, dn, dr, dv = 24, 4, 16, 8, 16
    q = orc.fill_normal((T, H, dn + dr), 1)
    kn = orc.fill_normal((T, H, dn), 2)
    kr = orc.fill_normal((T, dr), 3)
    v = orc.fill_normal((T, H, dv), 4)
    full = orc.causal_mha(q, kn, kr, v, 0.2, threads=1)
    qb, qe, kb, ke = shard_heads(H, H, world, rank)
    local = orc.causal_mha(np.ascontiguousarray(q[:, qb:qe]), np.ascontiguousarray(kn[:, kb:ke]), kr,
                           np.ascontiguousarray(v[:, kb:ke]), 0.2, threads=1)
    gathered = allgather_heads(torch.from_numpy(local))
    ok_heads = bool(np.array_equal(gathered.numpy(), full))
    b, e = shard_sequences(5, world, rank)
    mine = torch.zeros(5, dtype=torch.int32)
    mine[b:e] = 1
    dist.all_reduce(mine)
    ok_seq = bool((mine == 1).all())
    q_out.put((rank, ok_heads and ok_seq, f"heads {ok_heads}, sequences {ok_seq}"))
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharding_allgather_and_sequence_sharding_world2():
    from oracle import pyoracle
    pyoracle.build()
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    from tests.workloads import collect_ranks
    results = collect_ranks(procs, q_out, timeout=120)
    assert sorted(r[0] for r in results) == [0, 1]
