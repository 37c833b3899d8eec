"""Content addressing of a GPU-built two-tier pool: compressed blocks, per-layer digests, the pool id,
the agent shells and the records that bind them, computed the way the reference computes them, so that
a pool encoded by the kernels can be handed over as the reference's `SharedKVPool` / `AgentShell` material.

Followed here (host side, blake3 over canonical JSON):
  * `CompressedBlock::new`            proveKV/src/codec.rs:83-95   payload digest = blake3(payload) as hex
  * `PoolLayer::compute_digest`       proveKV/src/pool.rs:83-103   blake3 of {"layer_index", "key_digests", "value_digests"}
  * pool id                           proveKV/src/pool.rs:329-343  blake3 of {"layer_digests", "codebook_digest",
                                                                   "rotation_digest", "shape", "seed", "shared_codec"}
  * corpus layout and batch order     proveKV/src/pool.rs:246-266  per token a vector [layer][head][K d | V d];
                                                                   one FB2 blob per (layer, K|V), vectors token-major
  * pool manifest and build receipt   proveKV/src/pool.rs:345-383  (`records.PoolManifest`, `records.PoolBuildReceipt`)
  * `materialize_shell`               proveKV/src/shell.rs:148-379 one TQB1 blob per (layer, K|V); shell digest =
                                                                   blake3 of {"agent_id", "pool_digest",
                                                                   "layer_digests", "seed"}
  * injection traces                  proveKV/src/receipt.rs:217-241
`serde_json::json!` builds maps with sorted keys (the crate does not enable `preserve_order`) and
`to_string` writes them without spaces: `_canonical` below does the same.  Records that derive
`Serialize` keep their field order instead; `records.py` writes those.

Not reproduced: the codebook and rotation digests (fib-quant/src/codebook.rs:134-157 hashes the
serialised tables, profile and training report) are taken as strings from whoever owns the tables;
the page store, leases and authority checks stay with the reference.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field

import numpy as np

from . import _lib as L
from .codec import CODEC_FIB_K4_N32_BATCHED, turbo_batched_codec_id
from .pool import payload_batch_stride
from .records import (BlockInjectionTrace, CompressionPolicy, InjectionReceipt, KvTensorShape, PoolBuildReceipt,
                      PoolManifest, ShellManifest, ShellMaterializeReceipt, now_unix)

__all__ = ["CompressedBlock", "PoolLayer", "ShellLayer", "AgentShell", "KvTensorShape", "pool_id", "shell_digest",
           "build_shared_pool", "materialize_shell", "injection_receipt"]


def _blake3_hex(data: bytes) -> str:
    import blake3
    return blake3.blake3(data).hexdigest()


def _canonical(obj) -> bytes:
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode()


@dataclass
class CompressedBlock:
    """proveKV/src/codec.rs:70-108."""
    codec: str
    encoded_payload: bytes
    original_dim: int
    payload_digest: str = field(init=False)
    compressed_bytes: int = field(init=False)

    def __post_init__(self):
        self.compressed_bytes = len(self.encoded_payload)
        self.payload_digest = _blake3_hex(self.encoded_payload)

    def compression_ratio(self) -> float:
        return 0.0 if self.compressed_bytes == 0 else self.original_dim * 4 / self.compressed_bytes


@dataclass
class PoolLayer:
    """proveKV/src/pool.rs:44-103: one batched block per side."""
    layer_index: int
    key_blocks: list
    value_blocks: list
    block_digest: str = ""

    def compute_digest(self) -> str:
        return _blake3_hex(_canonical({
            "layer_index": self.layer_index,
            "key_digests": [b.payload_digest for b in self.key_blocks],
            "value_digests": [b.payload_digest for b in self.value_blocks],
        }))


def pool_id(layer_digests, codebook_digest: str, rotation_digest: str, shape: KvTensorShape, seed: int,
            shared_codec: str = CODEC_FIB_K4_N32_BATCHED) -> str:
    """proveKV/src/pool.rs:329-343."""
    return _blake3_hex(_canonical({
        "layer_digests": list(layer_digests), "codebook_digest": codebook_digest,
        "rotation_digest": rotation_digest, "shape": shape.as_json(), "seed": seed,
        "shared_codec": shared_codec}))


def shell_digest(agent_id: str, pool_digest: str, layer_digests, seed: int) -> str:
    """proveKV/src/shell.rs:322-337; an agent without tokens of its own hashes a fixed text instead (:158-161)."""
    layer_digests = list(layer_digests)
    if not layer_digests:
        return _blake3_hex(f"empty_shell:{agent_id}:{pool_digest}".encode())
    return _blake3_hex(_canonical({"agent_id": agent_id, "pool_digest": pool_digest,
                                   "layer_digests": layer_digests, "seed": seed}))


def _encode_layer_blobs(profile, tokens, shape: KvTensorShape, device):
    """One launch over the ``2 * layers`` batches of a ``[tokens][layer][head][K | V][dim]`` array, read in
    place through strides; returns the wire blob (header + records) of every (layer, side)."""
    import torch

    from .profiles import read_error_word

    x = np.ascontiguousarray(tokens, dtype=np.float32)
    T = x.shape[0]
    Lc, H, d = shape.num_layers, shape.num_kv_heads, shape.head_dim
    if x.ndim != 2 or x.shape[1] != Lc * H * 2 * d:
        raise ValueError(f"token vectors must be [tokens][{Lc * H * 2 * d}]")
    if d != profile.dim:
        raise ValueError("profile and shape disagree on head_dim")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    vpb, rec = T * H, profile.record_bytes
    stride = payload_batch_stride(vpb, rec)
    lay = L.Layout.make(n_tokens=T, n_heads=H, token_stride=Lc * H * 2 * d, head_stride=2 * d,
                        n_batches=(Lc, 2, 1), batch_stride=(H * 2 * d, d, 0))
    # the library launches on the current device and refuses a profile that lives on another one: the
    # data, the stream and the launch all belong to `dev`
    with torch.cuda.device(dev):
        x_dev = torch.from_numpy(x).to(dev)
        payload = torch.zeros((Lc, 2, stride), dtype=torch.uint8, device=dev)
        err = torch.full((1,), -1, dtype=torch.int64, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        profile.encode_dev(x_dev.data_ptr(), lay, payload.data_ptr(), stride, err.data_ptr(), stream)
        read_error_word(err.data_ptr(), stream)
        host = payload.cpu().numpy()
    header = profile.header(vpb)
    return [[header + host[li, side, :vpb * rec].tobytes() for side in range(2)] for li in range(Lc)]


def build_shared_pool(profile, corpus, shape: KvTensorShape, seed: int, codebook_digest: str,
                      rotation_digest: str, device=None, policy: CompressionPolicy | None = None,
                      built_at_unix: int | None = None) -> dict:
    """SharedKVPool::build (proveKV/src/pool.rs:160-400) with the encoding on the GPU.

    ``corpus``: f32 array ``[tokens][layers * kv_heads * 2 * head_dim]``, per token the reference's
    ``[layer][head][K | V][dim]`` vector (pool.rs:250-257).  All ``2 * layers`` batches are encoded
    by one launch; the result holds one FB2 blob per (layer, K|V) wrapped as the reference's blocks,
    the layer digests, the pool id, the manifest, and the build receipt with ``backend`` "gpu"."""
    policy = policy or CompressionPolicy.default_two_tier()
    policy.validate()
    shape.validate()
    if len(corpus) == 0:
        raise ValueError("empty corpus: cannot build pool from zero tokens")
    built_at_unix = now_unix() if built_at_unix is None else built_at_unix
    t0 = time.perf_counter()
    blobs = _encode_layer_blobs(profile, corpus, shape, device)
    fib_build_ms = int((time.perf_counter() - t0) * 1000)
    T, d = len(corpus), shape.head_dim
    layers, total = [], 0
    for li, (kb, vb) in enumerate(blobs):
        layer = PoolLayer(li, [CompressedBlock(policy.shared_codec, kb, d)], [CompressedBlock(policy.shared_codec, vb, d)])
        layer.block_digest = layer.compute_digest()
        total += len(kb) + len(vb)
        layers.append(layer)
    digests = [layer.block_digest for layer in layers]
    pid = pool_id(digests, codebook_digest, rotation_digest, shape, seed, policy.shared_codec)
    raw = shape.total_kv_bytes(T)
    manifest = PoolManifest.new(pid, shape, policy, T, shape.num_layers, total, raw, seed, built_at_unix)
    receipt = PoolBuildReceipt.new(pid, digests, codebook_digest, rotation_digest, T, fib_build_ms, total, raw,
                                   policy, seed, built_at_unix).with_backend("gpu")
    return {"pool_id": pid, "layers": layers, "layer_digests": digests, "num_tokens": T,
            "pool_size_bytes": total, "raw_size_bytes": raw, "seed": seed,
            "shared_codec": policy.shared_codec, "codebook_digest": codebook_digest,
            "rotation_digest": rotation_digest, "shape": shape.as_json(), "manifest": manifest, "receipt": receipt}


@dataclass
class ShellLayer:
    """proveKV/src/shell.rs:18-69: one batched turbo block per side; the digest has the pool layer's form."""
    layer_index: int
    key_blocks: list
    value_blocks: list
    block_digest: str = ""
    component_kind: object = "KeyValue"

    def compute_digest(self) -> str:
        return PoolLayer.compute_digest(self)


@dataclass
class AgentShell:
    """proveKV/src/shell.rs:72-90."""
    agent_id: str
    shell_manifest: ShellManifest
    unique_layers: list
    pool_digest: str


def materialize_shell(pool_manifest: PoolManifest, agent_id: str, agent_tokens, seed: int, profile=None,
                      device=None, materialized_at_unix: int | None = None):
    """`materialize_shell` (proveKV/src/shell.rs:148-379) with the turbo encode on the GPU.

    ``agent_tokens``: f32 ``[tokens][layers * kv_heads * 2 * head_dim]`` in the corpus layout.  Returns
    ``(AgentShell, ShellMaterializeReceipt)``.  The turbo profile comes from the policy in the pool's manifest
    and ``seed`` unless one is passed.  Non-finite inputs are refused before anything is encoded
    (shell.rs:215-221)."""
    from .codec import CorruptPayload, DimensionMismatch, _turbo_profile

    t0 = time.perf_counter()
    shape, policy = pool_manifest.shape, pool_manifest.policy
    tc = policy.turbo_config
    pid = pool_manifest.pool_id
    x = np.asarray(agent_tokens, dtype=np.float32)
    when = now_unix() if materialized_at_unix is None else materialized_at_unix
    if x.shape[0] == 0:
        manifest = ShellManifest.new(agent_id, pid, 0, pool_manifest.num_layers, 0, policy.shell_codec, seed, when,
                                     shape.head_dim, shape.num_kv_heads, tc)
        receipt = ShellMaterializeReceipt.new(agent_id, pid, shell_digest(agent_id, pid, [], seed), 0, 0,
                                              int((time.perf_counter() - t0) * 1000), when)
        return AgentShell(agent_id, manifest, [], pid), receipt
    expected = shape.num_layers * shape.num_kv_heads * shape.head_dim * 2
    if x.ndim != 2 or x.shape[1] != expected:
        raise DimensionMismatch(f"dimensionality mismatch: expected {expected}, got {x.shape[-1]}")
    bad = np.flatnonzero(~np.isfinite(x).all(axis=1))
    if bad.size:
        raise CorruptPayload(f"agent token {int(bad[0])} contains non-finite values")
    if profile is None:
        profile = _turbo_profile(shape.head_dim, tc.bits, tc.projections, tc.lossy_radii, seed)
    blobs = _encode_layer_blobs(profile, x, shape, device)
    codec_id = turbo_batched_codec_id(tc.bits, tc.lossy_radii)
    layers, total = [], 0
    for li, (kb, vb) in enumerate(blobs):
        layer = ShellLayer(li, [CompressedBlock(codec_id, kb, shape.head_dim)],
                           [CompressedBlock(codec_id, vb, shape.head_dim)])
        layer.block_digest = layer.compute_digest()
        total += len(kb) + len(vb)
        layers.append(layer)
    ms = int((time.perf_counter() - t0) * 1000)
    sd = shell_digest(agent_id, pid, [layer.block_digest for layer in layers], seed)
    manifest = ShellManifest.new(agent_id, pid, x.shape[0], shape.num_layers, total, policy.shell_codec, seed, when,
                                 shape.head_dim, shape.num_kv_heads, tc)
    manifest.component_kinds = [layer.component_kind for layer in layers]
    receipt = ShellMaterializeReceipt.new(agent_id, pid, sd, x.shape[0], total, ms, when)
    return AgentShell(agent_id, manifest, layers, pid), receipt


def injection_receipt(agent_id: str, pool_manifest: PoolManifest, pool_layer_digests, shell: AgentShell,
                      shell_digest_hex: str, injected_at_unix: int | None = None) -> InjectionReceipt:
    """The trace of one decode-and-patch of an agent's cache: per layer the pool block written at token 0,
    then the shell block written behind the shared prefix (proveKV/src/receipt.rs:217-261; the reference
    leaves the injection itself to a cache adapter, proveKV/src/pool.rs:422-433)."""
    traces = []
    for li, digest in enumerate(pool_layer_digests):
        traces.append(BlockInjectionTrace(li, "pool", digest, 0))
    for layer in shell.unique_layers:
        traces.append(BlockInjectionTrace(layer.layer_index, "shell", layer.block_digest,
                                          pool_manifest.num_shared_tokens))
    traces.sort(key=lambda t: (t.layer, t.source != "pool"))
    when = now_unix() if injected_at_unix is None else injected_at_unix
    receipt = InjectionReceipt.new(agent_id, pool_manifest.pool_id, shell_digest_hex, len(traces), traces, when)
    receipt.validate()
    return receipt
