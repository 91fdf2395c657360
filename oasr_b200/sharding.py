"""Utterance-level data parallelism: pack, deal packs to ranks, gather results on the host.

The encoder path has no exchange step between utterances, so N GPUs run N independent
shards (one process per GPU); the only communication is the final host-side gather of the
per-utterance token lists.  ``plan_packs`` restates the reference's packing partition
(PackingPartition.split, oasr/engine/batching/partition.py:100-127): sort by length, then
greedy gapless packs bounded by a post-subsampling frame budget (``max_packed_frames`` =
8192, oasr/engine/config.py:175).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence


def plan_packs(num_frames: Sequence[int], max_packed_frames: int = 8192, subsampling_rate: int = 4) -> List[List[int]]:
    """Utterance indices per pack, in the reference's order (ascending length, stable)."""
    order = sorted(range(len(num_frames)), key=lambda i: num_frames[i])
    budget = max(1, int(max_packed_frames))
    sr = max(1, int(subsampling_rate))
    packs: List[List[int]] = []
    cur: List[int] = []
    cur_sum = 0
    for i in order:
        tlen = max(1, int(num_frames[i]) // sr)
        if cur and cur_sum + tlen > budget:
            packs.append(cur)
            cur, cur_sum = [i], tlen
        else:
            cur.append(i)
            cur_sum += tlen
    if cur:
        packs.append(cur)
    return packs


def pack_cost(num_frames: Sequence[int], pack: Sequence[int], d_model: int = 512, ffn: int = 2048,
              subsampling_rate: int = 4) -> float:
    """Relative cost of a pack: dense work is linear in tokens, attention quadratic per utterance
    (12.06 MFLOP/token/layer at d 512 and 6*T^2*d per utterance for the attention products)."""
    dense_per_token = 2.0 * d_model * (4 * ffn + 8 * d_model)
    cost = 0.0
    for i in pack:
        t = max(1, int(num_frames[i]) // subsampling_rate)
        cost += t * dense_per_token + 6.0 * t * t * d_model
    return cost


def assign_packs(num_frames: Sequence[int], packs: Sequence[Sequence[int]], world_size: int, **cost_kw) -> List[List[int]]:
    """Deal packs to ranks, longest-processing-time first; returns pack indices per rank.
    Deterministic: every rank computes the same plan from the same lengths, no communication."""
    costs = [pack_cost(num_frames, p, **cost_kw) for p in packs]
    order = sorted(range(len(packs)), key=lambda j: (-costs[j], j))
    load = [0.0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for j in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        out[r].append(j)
        load[r] += costs[j]
    for r in range(world_size):
        out[r].sort()
    return out


def gather_results(local: Dict[int, List[int]], num_utterances: int, group=None) -> Optional[List[List[int]]]:
    """Collect ``{utterance index: tokens}`` from every rank on rank 0 (host-side object gather;
    works on gloo and nccl groups).  Rank 0 returns the token lists in utterance order and checks
    that every utterance arrived exactly once; the other ranks return None."""
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        merged = [local]
        rank = 0
    else:
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        bucket = [None] * world if rank == 0 else None
        dist.gather_object(local, bucket, dst=0, group=group)
        merged = bucket
    if rank != 0:
        return None
    out: List[Optional[List[int]]] = [None] * num_utterances
    for part in merged:
        for idx, toks in part.items():
            if out[idx] is not None:
                raise RuntimeError(f"utterance {idx} was processed by more than one rank")
            out[idx] = list(toks)
    missing = [i for i, t in enumerate(out) if t is None]
    if missing:
        raise RuntimeError(f"utterances {missing[:8]} were not processed by any rank")
    return out  # type: ignore[return-value]
