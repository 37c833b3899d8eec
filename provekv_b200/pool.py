"""Layouts of the two-tier pool: how the batches the reference builds per
(layer, K|V) map onto framework KV tensors, and the fused decode-and-patch
position map.

The reference gathers, per layer and per side (K or V), the vectors of all
tokens and heads in token-major, head-minor order (proveKV/src/pool.rs:246-257,
shell.rs:250-262) and patches decoded vectors into a cache tensor shaped
``(1, H, T, d)`` per layer at ``pos = t`` for shared tokens and
``pos = n_shared + agent * n_unique + t`` for agent tokens
(proveKV/scripts/ppl_validate_multi_agent.py:226-271).  Here one kernel launch
covers every (agent, layer, K|V) batch, reading or writing the framework tensor
in place through strides, so no gather / relayout copies exist.

Tensor convention used by the helpers: ``kv[agent][layer][side][head][token][dim]``
(the per-layer ``(H, T, d)`` block is exactly the HF cache layout of one batch
element), f32, contiguous.
"""
from __future__ import annotations

from dataclasses import dataclass

from ._lib import Layout


@dataclass(frozen=True)
class KvShape:
    """Model-side KV geometry (proveKV/src/shape.rs)."""
    num_layers: int
    num_kv_heads: int
    head_dim: int

    def vectors(self, n_tokens: int, n_agents: int = 1) -> int:
        return n_agents * self.num_layers * 2 * self.num_kv_heads * n_tokens


SMOLLM2_1_7B = KvShape(24, 32, 64)
QWEN25_0_5B = KvShape(24, 2, 64)
LLAMA3_8B = KvShape(32, 8, 128)


def kv_tensor_layout(shape: KvShape, n_agents: int, n_tokens: int, token_capacity: int | None = None,
                     first_token: int = 0, n_replicas: int = 1, replica_stride: int = 0) -> Layout:
    """Layout of ``n_tokens`` tokens starting at ``first_token`` inside a tensor
    ``[n_agents][layers][2][heads][token_capacity][dim]``: one batch per (agent, layer, side)."""
    cap = n_tokens if token_capacity is None else token_capacity
    if first_token + n_tokens > cap:
        raise ValueError("tokens do not fit the cache")
    d, h = shape.head_dim, shape.num_kv_heads
    side = h * cap * d
    layer = 2 * side
    agent = shape.num_layers * layer
    return Layout.make(base=first_token * d, n_batches=(n_agents, shape.num_layers, 2),
                       batch_stride=(agent, layer, side), n_tokens=n_tokens, n_heads=h,
                       token_stride=d, head_stride=cap * d, n_replicas=n_replicas,
                       replica_stride=replica_stride)


def payload_batch_stride(vectors_per_batch: int, record_bytes: int) -> int:
    """Bytes between the payloads of consecutive batches: records, rounded up to 16."""
    return (vectors_per_batch * record_bytes + 15) // 16 * 16


def agent_patch_position(n_shared: int, n_unique: int, agent: int) -> int:
    """First cache position of an agent's unique tokens
    (proveKV/scripts/ppl_validate_multi_agent.py:258)."""
    return n_shared + agent * n_unique
