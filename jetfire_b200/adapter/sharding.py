"""Partition of the decode hot path over the GPUs of one node, and the one exchange it needs.

Every (batch element, KV head) pair is independent until the per-head outputs are
concatenated, so the path shards without any data-path collective: KV heads first (query
heads follow in groups of ``H_q / H_kv``, which is vLLM's tensor-parallel head layout --
the reference sees only local heads, tests/test_runtime_edge_cases.py:29-48 of JetFire),
then batch elements once the KV heads run out.  Each rank owns the packed cache, the host
mirror and the correction threads of its shard.  The only exchange is the gather of the
per-head outputs into the ``(B, H_q * 128)`` layout, a few KB per layer-step.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Shard:
    rank: int
    kv_start: int      # first KV head of this rank
    kv_count: int
    q_start: int       # first query head (= kv_start * group)
    q_count: int
    b_start: int       # first batch element
    b_count: int


def shard_plan(H_q: int, H_kv: int, B: int, world: int) -> list[Shard]:
    """KV heads are split over ``min(world, H_kv)`` head shards; the remaining factor of
    ``world`` splits the batch.  Raises ValueError when the sizes do not divide."""
    if world <= 0 or H_q % H_kv:
        raise ValueError("bad geometry")
    group = H_q // H_kv
    head_shards = min(world, H_kv)
    if H_kv % head_shards or world % head_shards:
        raise ValueError(f"{H_kv} KV heads cannot be split over {world} ranks")
    batch_shards = world // head_shards
    if B % batch_shards:
        raise ValueError(f"batch {B} cannot be split {batch_shards} ways once the KV heads are exhausted")
    kv_per, b_per = H_kv // head_shards, B // batch_shards
    plan = []
    for r in range(world):
        hs, bs = r % head_shards, r // head_shards
        plan.append(Shard(r, hs * kv_per, kv_per, hs * kv_per * group, kv_per * group, bs * b_per, b_per))
    return plan


def cpu_threads_per_rank(cores: int, world: int) -> int:
    """Correction workers per rank: the host cores are shared by the ranks of a node."""
    return max(1, cores // max(world, 1))


def resolve_numa_node(configured: int, device_node: int, node_count: int) -> int:
    """Memory node for a rank's host mirrors and correction workers, -1 for none.
    ``configured``: -2 = the GPU's own node when the host has more than one and says where the
    GPU sits, -1 = none, otherwise the node itself (ignored on a host that lacks it)."""
    if configured == -1 or node_count <= 1:
        return -1
    if configured == -2:
        return device_node if 0 <= device_node < node_count else -1
    return configured if 0 <= configured < node_count else -1


def workers_on_node(want: int, node_cpus: int, ranks_on_node: int) -> int:
    """Correction workers of a rank that is confined to one memory node: that node's processors
    are shared by the ranks placed there."""
    return max(1, min(want, node_cpus // max(ranks_on_node, 1)))


def gather_outputs(local_out: torch.Tensor, plan: list[Shard], B: int, H_q: int, group=None) -> torch.Tensor:
    """All-gather ``local_out (b_count, q_count, 128)`` of every rank into ``(B, H_q * 128)``.
    One collective (NCCL on GPUs, gloo on CPU); shards are equal-sized by construction."""
    world = len(plan)
    if world == 1:
        return local_out.reshape(B, H_q * 128)
    local_out = local_out.contiguous()
    gathered = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(gathered, local_out, group=group)
    full = torch.empty(B, H_q, 128, dtype=local_out.dtype, device=local_out.device)
    for s in plan:
        full[s.b_start:s.b_start + s.b_count, s.q_start:s.q_start + s.q_count] = gathered[s.rank]
    return full.reshape(B, H_q * 128)
