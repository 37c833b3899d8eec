"""Content addressing of a GPU-built shared pool: compressed blocks, per-layer digests and the pool id,
computed the way the reference computes them, so that a pool encoded by the kernels can be handed
over as the reference's `SharedKVPool` material.

Followed here (host side, blake3 over canonical JSON):
  * `CompressedBlock::new`            proveKV/src/codec.rs:83-95   payload digest = blake3(payload) as hex
  * `PoolLayer::compute_digest`       proveKV/src/pool.rs:83-103   blake3 of {"layer_index", "key_digests", "value_digests"}
  * pool id                           proveKV/src/pool.rs:329-343  blake3 of {"layer_digests", "codebook_digest",
                                                                   "rotation_digest", "shape", "seed", "shared_codec"}
  * corpus layout and batch order     proveKV/src/pool.rs:246-266  per token a vector [layer][head][K d | V d];
                                                                   one FB2 blob per (layer, K|V), vectors token-major
`serde_json::json!` builds maps with sorted keys (the crate does not enable `preserve_order`) and
`to_string` writes them without spaces: `_canonical` below does the same.

Not reproduced: the codebook and rotation digests (fib-quant/src/codebook.rs:134-157 hashes the
serialised tables, profile and training report) are taken as strings from whoever owns the tables;
receipts and the page store stay with the reference.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

import numpy as np

from . import _lib as L
from .codec import CODEC_FIB_K4_N32_BATCHED
from .pool import payload_batch_stride

__all__ = ["CompressedBlock", "PoolLayer", "KvTensorShape", "pool_id", "build_shared_pool"]


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


@dataclass(frozen=True)
class KvTensorShape:
    """proveKV/src/shape.rs:20-34; `attention_type` serialises in lower case (:7)."""
    attention_type: str
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    hidden_size: int

    def as_json(self) -> dict:
        return {"attention_type": self.attention_type.lower(), "num_layers": self.num_layers,
                "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
                "hidden_size": self.hidden_size}

    def total_kv_bytes(self, num_tokens: int) -> int:
        """shape.rs:104-113: layers x 2 x kv heads x head_dim x tokens f32 values."""
        return self.num_layers * 2 * self.num_kv_heads * self.head_dim * num_tokens * 4


def pool_id(layer_digests, codebook_digest: str, rotation_digest: str, shape: KvTensorShape, seed: int,
            shared_codec: str = CODEC_FIB_K4_N32_BATCHED) -> str:
    """proveKV/src/pool.rs:329-343."""
    return _blake3_hex(_canonical({
        "layer_digests": list(layer_digests), "codebook_digest": codebook_digest,
        "rotation_digest": rotation_digest, "shape": shape.as_json(), "seed": seed,
        "shared_codec": shared_codec}))


def build_shared_pool(profile, corpus, shape: KvTensorShape, seed: int, codebook_digest: str,
                      rotation_digest: str, device=None) -> dict:
    """SharedKVPool::build (proveKV/src/pool.rs:160-400) with the encoding on the GPU.

    ``corpus``: f32 array ``[tokens][layers * kv_heads * 2 * head_dim]``, per token the reference's
    ``[layer][head][K | V][dim]`` vector (pool.rs:250-257).  All ``2 * layers`` batches are encoded
    by one launch reading the corpus in place through strides; the result holds one FB2 blob per
    (layer, K|V) wrapped as the reference's blocks, the layer digests and the pool id."""
    import torch

    x = np.ascontiguousarray(corpus, dtype=np.float32)
    T = x.shape[0]
    Lc, H, d = shape.num_layers, shape.num_kv_heads, shape.head_dim
    if x.ndim != 2 or x.shape[1] != Lc * H * 2 * d:
        raise ValueError(f"corpus must be [tokens][{Lc * H * 2 * d}]")
    if d != profile.dim:
        raise ValueError("profile and shape disagree on head_dim")
    if T == 0:
        raise ValueError("empty corpus")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    x_dev = torch.from_numpy(x).to(dev)
    vpb, rec = T * H, profile.record_bytes
    stride = payload_batch_stride(vpb, rec)
    payload = torch.zeros((Lc, 2, stride), dtype=torch.uint8, device=dev)
    err = torch.full((1,), -1, dtype=torch.int64, device=dev)
    lay = L.Layout.make(n_tokens=T, n_heads=H, token_stride=Lc * H * 2 * d, head_stride=2 * d,
                        n_batches=(Lc, 2, 1), batch_stride=(H * 2 * d, d, 0))
    stream = torch.cuda.current_stream(dev).cuda_stream
    profile.encode_dev(x_dev.data_ptr(), lay, payload.data_ptr(), stride, err.data_ptr(), stream)
    from .profiles import read_error_word
    read_error_word(err.data_ptr(), stream)
    host = payload.cpu().numpy()
    header = profile.header(vpb)
    layers, total = [], 0
    for li in range(Lc):
        blocks = [CompressedBlock(CODEC_FIB_K4_N32_BATCHED, header + host[li, side, :vpb * rec].tobytes(), d)
                  for side in range(2)]
        layer = PoolLayer(li, [blocks[0]], [blocks[1]])
        layer.block_digest = layer.compute_digest()
        total += blocks[0].compressed_bytes + blocks[1].compressed_bytes
        layers.append(layer)
    digests = [layer.block_digest for layer in layers]
    pid = pool_id(digests, codebook_digest, rotation_digest, shape, seed)
    return {"pool_id": pid, "layers": layers, "layer_digests": digests, "num_tokens": T,
            "pool_size_bytes": total, "raw_size_bytes": shape.total_kv_bytes(T), "seed": seed,
            "shared_codec": CODEC_FIB_K4_N32_BATCHED, "codebook_digest": codebook_digest,
            "rotation_digest": rotation_digest, "shape": shape.as_json()}
