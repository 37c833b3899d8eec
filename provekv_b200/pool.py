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


@dataclass(frozen=True)
class TwoTierPlan:
    """Where one rank's part of the two-tier pool lives and which kernel launch covers it.

    The reference builds one cold pool of the shared prefix (fib-quant, one batch per (layer, K|V),
    proveKV/src/pool.rs:246-309), one hot shell per agent (turbo-quant, proveKV/src/shell.rs:250-311,
    examples/prove_kv_multi_agent_shell.rs:272-331) and patches both into the agents' caches
    (proveKV/scripts/ppl_validate_multi_agent.py:226-271): prefix token t at position t of every
    cache, agent a's token t at ``n_shared + a * n_unique + t`` of its own cache, each cache holding
    ``n_shared + n_agents * n_unique`` positions.

    ``shard = "agent"``: the rank owns a block of agents (their shells and caches) and encodes a block
    of the prefix's layers; the FB2 payload of the other layers arrives by an all-gather, and the
    rank decodes the whole pool into its agents' caches.  ``shard = "layer"``: the rank owns a block
    of layers of everything; nothing is exchanged.

    Tensors (f32, contiguous): prefix ``[enc_layers][2][H][n_shared][d]``, shells
    ``[agents][dec_layers][2][H][n_unique][d]``, caches ``[agents][dec_layers][2][H][cache_tokens][d]``.
    """
    shape: KvShape
    n_agents: int
    n_shared: int
    n_unique: int
    world_size: int = 1
    rank: int = 0
    shard: str = "agent"

    def __post_init__(self):
        if self.shard not in ("agent", "layer"):
            raise ValueError("shard must be 'agent' or 'layer'")
        if not 0 <= self.rank < self.world_size:
            raise ValueError("bad rank / world_size")

    @staticmethod
    def _block(n: int, world: int, rank: int) -> range:
        return range(n * rank // world, n * (rank + 1) // world)

    @property
    def cache_tokens(self) -> int:
        return self.n_shared + self.n_agents * self.n_unique

    @property
    def agents(self) -> range:
        if self.shard == "agent":
            return self._block(self.n_agents, self.world_size, self.rank)
        return range(self.n_agents)

    @property
    def enc_layers(self) -> range:
        """Prefix layers this rank encodes."""
        return self._block(self.shape.num_layers, self.world_size, self.rank)

    @property
    def dec_layers(self) -> range:
        """Layers present in this rank's shells and caches."""
        return range(self.shape.num_layers) if self.shard == "agent" else self.enc_layers

    def _sub(self, layers: range) -> KvShape:
        return KvShape(len(layers), self.shape.num_kv_heads, self.shape.head_dim)

    @property
    def agent_cache_elems(self) -> int:
        s = self.shape
        return len(self.dec_layers) * 2 * s.num_kv_heads * self.cache_tokens * s.head_dim

    def prefix_vectors(self, layers: range) -> int:
        return self._sub(layers).vectors(self.n_shared)

    def shell_vectors(self) -> int:
        return self._sub(self.dec_layers).vectors(self.n_unique, len(self.agents))

    def prefix_encode_layout(self) -> Layout:
        return kv_tensor_layout(self._sub(self.enc_layers), 1, self.n_shared)

    def prefix_decode_layout(self) -> Layout:
        """One decode of the pool's dec_layers, written into every owned agent's cache."""
        return kv_tensor_layout(self._sub(self.dec_layers), 1, self.n_shared,
                                token_capacity=self.cache_tokens, first_token=0,
                                n_replicas=len(self.agents), replica_stride=self.agent_cache_elems)

    def shell_encode_layout(self) -> Layout:
        return kv_tensor_layout(self._sub(self.dec_layers), len(self.agents), self.n_unique)

    def shell_decode_layout(self) -> Layout:
        """Agent a (global index) lands at position n_shared + a * n_unique of its own cache: the
        step from one agent's batches to the next is one cache plus n_unique positions."""
        s, d = self._sub(self.dec_layers), self.shape.head_dim
        L = kv_tensor_layout(s, len(self.agents), self.n_unique, token_capacity=self.cache_tokens,
                             first_token=agent_patch_position(self.n_shared, self.n_unique, self.agents.start)
                             if len(self.agents) else 0)
        L.batch_stride[0] = self.agent_cache_elems + self.n_unique * d
        return L
