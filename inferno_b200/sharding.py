"""How the attention path is split over the GPUs of one box, and the one collective it needs.

Attention rows are independent per (sequence, head) and GQA groups are independent per KV head, so
  * batched decode shards by sequence: every rank owns whole sequences and their pages, no exchange;
  * prefill and MLA shard by head group: rank r owns q heads [r*Hq/N, (r+1)*Hq/N) and the KV heads they
    read, and the attention output is all-gathered (NCCL over NVLink on GPUs, gloo on CPU).
The reference has no multi-device path; this module is the whole of it here.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_heads(q_heads: int, kv_heads: int, world: int, rank: int):
    """(q_begin, q_end, kv_begin, kv_end) of rank's head group; groups are never split across ranks."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if kv_heads % world or q_heads % kv_heads:
        raise ValueError(f"{kv_heads} KV heads (of {q_heads} q heads) do not split over {world} ranks")
    kv_per, group = kv_heads // world, q_heads // kv_heads
    return rank * kv_per * group, (rank + 1) * kv_per * group, rank * kv_per, (rank + 1) * kv_per


def shard_sequences(batch: int, world: int, rank: int):
    """[begin, end) of the sequences rank owns: contiguous blocks, sizes differing by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(batch, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def balanced_sequence_order(lengths, world: int):
    """Order of a batch in which the contiguous blocks of shard_sequences hold about the same number of cached keys.

    Decode time is proportional to the keys a rank streams, so a batch split in arrival order leaves every rank
    waiting for the one that drew the long contexts.  Longest first, each sequence goes to the rank with the fewest
    keys so far that still has room in its block, then single exchanges with the fullest rank; the result lists rank 0's sequences, then rank 1's, and so on."""
    n = len(lengths)
    if world <= 0:
        raise ValueError(f"bad world size {world}")
    room = [shard_sequences(n, world, r)[1] - shard_sequences(n, world, r)[0] for r in range(world)]
    load = [0] * world
    owned = [[] for _ in range(world)]
    for i in sorted(range(n), key=lambda i: (-int(lengths[i]), i)):
        r = min((r for r in range(world) if len(owned[r]) < room[r]), key=lambda r: (load[r], r))
        owned[r].append(i)
        load[r] += int(lengths[i])
    # exchange single sequences between the fullest rank and the others while that lowers the larger of the two loads
    for _ in range(4 * n):
        hi = max(range(world), key=lambda r: (load[r], -r))
        best = None
        for lo in range(world):
            if lo == hi:
                continue
            for a in owned[hi]:
                for b in owned[lo]:
                    d = int(lengths[a]) - int(lengths[b])
                    if d > 0 and load[lo] + d < load[hi] and (best is None or max(load[hi] - d, load[lo] + d) < best[0]):
                        best = (max(load[hi] - d, load[lo] + d), lo, a, b, d)
        if best is None:
            break
        _, lo, a, b, d = best
        owned[hi][owned[hi].index(a)] = b
        owned[lo][owned[lo].index(b)] = a
        load[hi] -= d
        load[lo] += d
    return [i for r in range(world) for i in sorted(owned[r])]


def allgather_heads(local_out: torch.Tensor, group=None) -> torch.Tensor:
    """local_out [tokens, heads/N, dim] on every rank -> [tokens, heads, dim] (heads in rank order).

    One all-gather into a [N, tokens, heads/N, dim] buffer, then a strided view puts the gathered
    dimension in the middle; the copy to contiguous happens on the device."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    local_out = local_out.contiguous()
    t, h, d = local_out.shape
    gathered = torch.empty((world * t, h, d), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered, local_out, group=group)  # rank-major concatenation along dim 0
    return gathered.view(world, t, h, d).permute(1, 0, 2, 3).reshape(t, world * h, d)
