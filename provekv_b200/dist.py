"""Multi-GPU plumbing: one process per GPU, no collective on the codec path.

Every vector is independent and the reference batches per (layer, K|V) and per
agent (proveKV/src/pool.rs:299-304, examples/prove_kv_multi_agent_shell.rs:272-331),
so the work shards by agent or by layer with no exchange.  The only transfer is
the replication of the compressed cold pool (FB2 payload bytes) to every GPU that
serves agents: one ``torch.distributed.broadcast`` (NCCL over NVLink on GPUs, gloo
in the CPU tests) into each rank's local memory; decode kernels then read local
memory only.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_range(n_items: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) block of ``n_items`` for ``rank``; sizes differ by at most one."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("bad rank / world_size")
    return n_items * rank // world_size, n_items * (rank + 1) // world_size


def shard_agents(n_agents: int, world_size: int, rank: int) -> range:
    """Agents owned by ``rank`` (configs sharded by agent)."""
    lo, hi = shard_range(n_agents, world_size, rank)
    return range(lo, hi)


def shard_layers(n_layers: int, world_size: int, rank: int) -> range:
    """Layers owned by ``rank`` (long-context config sharded by layer)."""
    lo, hi = shard_range(n_layers, world_size, rank)
    return range(lo, hi)


def all_shards(n_items: int, world_size: int) -> List[Tuple[int, int]]:
    return [shard_range(n_items, world_size, r) for r in range(world_size)]


def broadcast_pool(payload, src: int = 0, group=None):
    """Replicate the compressed pool tensor (uint8) from ``src`` to every rank, in place."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(payload, src=src, group=group)
    return payload


def gather_layer_shards(local_payload, world_size: int, group=None):
    """All-gather equally sized per-rank pool shards (pool encoded layer-sharded) so every
    rank ends up with the whole pool; returns the list of per-rank tensors."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or world_size == 1:
        return [local_payload]
    out = [torch.empty_like(local_payload) for _ in range(world_size)]
    dist.all_gather(out, local_payload, group=group)
    return out


def max_over_ranks(values: Sequence[float], device=None) -> List[float]:
    """Element-wise max of per-rank timings (the reported time is the slowest rank's)."""
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]
