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


def all_gather_pool(local_payload, pool_payload, group=None, async_op=False):
    """Layer-sharded pool build: every rank has encoded an equal, contiguous block of the pool's
    batches (``local_payload``); afterwards ``pool_payload`` (world_size times as large, rank order
    = layer order) holds the whole pool in every rank's own memory.  With one rank the local block
    is the pool and is copied unless both arguments are the same tensor.  ``async_op``: returns the
    collective's work handle (None with one rank); ``wait()`` on it before the pool is read."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if pool_payload.numel() != local_payload.numel() * dist.get_world_size(group):
            raise ValueError("the pool must be world_size equal blocks")
        work = dist.all_gather_into_tensor(pool_payload.view(-1), local_payload.view(-1), group=group,
                                           async_op=async_op)
        return work if async_op else pool_payload
    if pool_payload.data_ptr() != local_payload.data_ptr():
        pool_payload.view(-1).copy_(local_payload.view(-1))
    return None if async_op else pool_payload


def gpu_numa_cpus(pci_bus_id: str, sysfs: str = "/sys/bus/pci/devices"):
    """CPUs of the NUMA node a GPU hangs off, from sysfs (``local_cpulist`` of the PCI device);
    an empty list when the platform does not say (virtual machines often report node -1)."""
    import os

    dev = os.path.join(sysfs, pci_bus_id.lower())
    try:
        with open(os.path.join(dev, "numa_node")) as f:
            if int(f.read().strip()) < 0:
                return []
        with open(os.path.join(dev, "local_cpulist")) as f:
            text = f.read().strip()
    except (OSError, ValueError):
        return []
    cpus = []
    for part in text.split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus += list(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_rank_to_gpu_numa(device_index: int):
    """Pin the calling process (its copy-issuing threads and the pages of the pinned buffers it
    allocates afterwards) to the CPUs next to its GPU, so that several ranks on one host do not
    pull their host<->device copies through one socket.  Returns the CPU list used ([] = left
    unchanged: no NUMA information, or the intersection with the allowed CPUs is empty)."""
    import os

    import torch

    props = torch.cuda.get_device_properties(device_index)
    try:
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    except AttributeError:
        return []
    cpus = sorted(set(gpu_numa_cpus(bus)) & set(os.sched_getaffinity(0)))
    if cpus:
        os.sched_setaffinity(0, cpus)
    return cpus


def max_over_ranks(values: Sequence[float], device=None) -> List[float]:
    """Element-wise max of per-rank timings (the reported time is the slowest rank's)."""
    import torch
    import torch.distributed as dist

    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]
