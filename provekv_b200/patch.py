"""Framework side of decode-and-patch: the kv binary files the reference's multi-agent example
writes, and patching a live per-layer KV cache (f32, fp16 or bf16) straight from compressed records.

The reference decodes a pool or shell to flat f32 lists in ``[token][head][dim]`` order, writes them
to a kv binary file (proveKV/examples/prove_kv_multi_agent_shell.rs:106-122), reads that file back
in Python (proveKV/scripts/ppl_validate_multi_agent.py:202-224) and copies the values token by token
into each layer's ``(1, H, T, d)`` cache tensor with ``dtype=k.dtype``
(ppl_validate_multi_agent.py:226-271), which is then installed in a ``DynamicCache`` (:282-293).
`patch_cache` does the last three steps in one kernel launch per cache tensor: the decode kernel
writes every vector at its ``[head][pos]`` slot of the tensor it is given, rounding to the tensor's
element type in the store.
"""
from __future__ import annotations

import json
import struct
from typing import Iterable, Sequence

import numpy as np

from . import _lib as L
from .pool import payload_batch_stride

__all__ = ["write_kv_binary", "read_kv_binary", "dst_dtype_of", "cache_tensor_layout", "cache_layers",
           "CachePlan", "plan_cache", "patch_cache"]


def write_kv_binary(path, manifest: dict, layers: Sequence[tuple[np.ndarray, np.ndarray]]) -> None:
    """u64 LE manifest length, the manifest as JSON, then per layer: u32 LE count + K values as
    f32 LE, u32 LE count + V values (prove_kv_multi_agent_shell.rs:106-122)."""
    blob = json.dumps(manifest, separators=(",", ":")).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for k, v in layers:
            for side in (k, v):
                a = np.ascontiguousarray(side, dtype="<f4").reshape(-1)
                if a.size >= 1 << 32:
                    raise ValueError("a kv binary side holds at most 2^32 - 1 values")
                f.write(struct.pack("<I", a.size))
                f.write(a.tobytes())


def read_kv_binary(path):
    """Inverse of `write_kv_binary`; returns ``(manifest, {layer: (k, v)}, num_layers,
    num_kv_heads, head_dim)`` with k, v flat f32 arrays in ``[token][head][dim]`` order, the tuple
    ppl_validate_multi_agent.py:202-224 returns.  Truncated files raise ValueError."""
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise ValueError("kv binary: missing manifest length")
        (n,) = struct.unpack("<Q", head)
        blob = f.read(n)
        if len(blob) != n:
            raise ValueError("kv binary: truncated manifest")
        manifest = json.loads(blob.decode())
        num_layers, heads, dim = manifest["num_layers"], manifest["num_kv_heads"], manifest["head_dim"]
        layers = {}
        for layer in range(num_layers):
            sides = []
            for _ in range(2):
                cnt = f.read(4)
                if len(cnt) != 4:
                    raise ValueError(f"kv binary: layer {layer} is missing")
                (m,) = struct.unpack("<I", cnt)
                raw = f.read(4 * m)
                if len(raw) != 4 * m:
                    raise ValueError(f"kv binary: layer {layer} is truncated")
                sides.append(np.frombuffer(raw, dtype="<f4").astype(np.float32))
            layers[layer] = (sides[0], sides[1])
    return manifest, layers, num_layers, heads, dim


def dst_dtype_of(tensor) -> int:
    """PKV_DST_* code of a torch tensor's element type."""
    import torch
    table = {torch.float32: L.DST_F32, torch.float16: L.DST_F16, torch.bfloat16: L.DST_BF16}
    if tensor.dtype not in table:
        raise TypeError(f"cache tensors must be float32, float16 or bfloat16, not {tensor.dtype}")
    return table[tensor.dtype]


def cache_tensor_layout(tensor, n_tokens: int, pos0: int) -> L.Layout:
    """Layout of one batch (token-major, head-minor vector order, pool.rs:246-257) written into a
    ``(1, H, T, d)`` or ``(H, T, d)`` cache tensor at token positions ``pos0 .. pos0 + n_tokens``
    (ppl_validate_multi_agent.py:247-262).  Strides are taken from the tensor, so a view with a
    larger token capacity works as long as the ``d`` values of a vector are contiguous."""
    if tensor.dim() == 4:
        if tensor.shape[0] != 1:
            raise ValueError("a 4-d cache tensor must have batch size 1")
        tensor = tensor[0]
    if tensor.dim() != 3:
        raise ValueError("cache tensor must be (1, H, T, d) or (H, T, d)")
    heads, cap, _ = tensor.shape
    if tensor.stride(2) != 1:
        raise ValueError("the values of a vector must be contiguous in the cache")
    if pos0 < 0 or pos0 + n_tokens > cap:
        raise ValueError(f"positions {pos0}..{pos0 + n_tokens} do not fit a cache of {cap} tokens")
    lay = L.Layout()
    lay.base = pos0 * tensor.stride(1)
    lay.batch_stride[0] = lay.batch_stride[1] = lay.batch_stride[2] = 0
    lay.n_batches[0] = lay.n_batches[1] = lay.n_batches[2] = 1
    lay.token_stride = tensor.stride(1)
    lay.head_stride = tensor.stride(0)
    lay.replica_stride = 0
    lay.n_tokens, lay.n_heads, lay.n_replicas = n_tokens, heads, 1
    return lay


def cache_layers(cache) -> list[tuple]:
    """(keys, values) per layer of a transformers ``DynamicCache`` (``cache.layers[i].keys`` /
    ``.values``, the fields ppl_validate_multi_agent.py:288-293 fills), of a
    ``{layer: {"k": ..., "v": ...}}`` dict (:264) or of a list of pairs."""
    if hasattr(cache, "layers"):
        return [(layer.keys, layer.values) for layer in cache.layers]
    if isinstance(cache, dict):
        return [(cache[i]["k"], cache[i]["v"]) for i in sorted(cache)]
    return [tuple(pair) for pair in cache]


class CachePlan:
    """Where the tensors of a cache sit relative to the lowest one: what one decode-and-patch launch
    over all of them needs.  Build it once per cache (`plan_cache`) and pass it to `patch_cache`;
    it stays valid while the cache's tensors are not reallocated."""

    def __init__(self, base_ptr: int, offsets, dst_dtype: int, heads: int, token_stride: int,
                 head_stride: int, capacity: int, n_layers: int):
        self.base_ptr, self.offsets, self.dst_dtype = base_ptr, offsets, dst_dtype
        self.heads, self.token_stride, self.head_stride = heads, token_stride, head_stride
        self.capacity, self.n_layers = capacity, n_layers


def plan_cache(cache) -> CachePlan | None:
    """A `CachePlan` if every tensor of the cache has the same shape, strides, element type and
    device and the distances between them are whole multiples of 16 bytes; otherwise None (then
    `patch_cache` launches once per tensor)."""
    import torch
    layers = cache_layers(cache)
    tensors = [t for pair in layers for t in pair]
    first = tensors[0]
    if any(t.shape != first.shape or t.stride() != first.stride() or t.dtype != first.dtype or
           t.device != first.device for t in tensors):
        return None
    view = first[0] if first.dim() == 4 else first
    if view.dim() != 3 or view.stride(2) != 1:
        return None
    esize = first.element_size()
    base = min(t.data_ptr() for t in tensors)
    if base % 16 or any((t.data_ptr() - base) % 16 for t in tensors):
        return None
    offsets = torch.tensor([(t.data_ptr() - base) // esize for t in tensors], dtype=torch.int64,
                           device=first.device)
    return CachePlan(base, offsets, dst_dtype_of(first), view.shape[0], view.stride(1), view.stride(0),
                     view.shape[1], len(layers))


def patch_cache(profile, payload, cache, n_tokens: int, pos0: int, err, stream: int = 0,
                plan: CachePlan | None = None) -> int:
    """Decode ``payload`` into the cache in place: one launch for the whole cache when its tensors
    are alike (``plan``, or `plan_cache(cache)` when none is given), else one per tensor.

    ``payload``: uint8 device tensor ``[layers][2][stride]`` of records without wire headers, batch
    (layer, side) at ``stride = payload_batch_stride(n_tokens * H, record_bytes)``.  ``cache``: see
    `cache_layers`; every tensor lives on the payload's device.  ``err``: the device error word
    (uint64 tensor of one element, reset by the caller); read it with `read_error_word` after the
    stream has run.  Returns the number of launches."""
    layers = cache_layers(cache)
    rec = profile.record_bytes
    heads = (layers[0][0][0] if layers[0][0].dim() == 4 else layers[0][0]).shape[0]
    stride = payload_batch_stride(n_tokens * heads, rec)
    if payload.dim() != 3 or payload.shape[0] != len(layers) or payload.shape[1] != 2 or payload.shape[2] != stride:
        raise ValueError(f"payload must be [layers={len(layers)}][2][{stride}] bytes")
    if plan is None:
        plan = plan_cache(cache)
    if plan is not None:
        if plan.n_layers != len(layers) or plan.heads != heads:
            raise ValueError("the plan was made for another cache")
        if pos0 < 0 or pos0 + n_tokens > plan.capacity:
            raise ValueError(f"positions {pos0}..{pos0 + n_tokens} do not fit a cache of {plan.capacity} tokens")
        lay = L.Layout()
        lay.base = pos0 * plan.token_stride
        lay.batch_stride[0] = lay.batch_stride[1] = lay.batch_stride[2] = 0
        lay.n_batches[0], lay.n_batches[1], lay.n_batches[2] = len(layers), 2, 1
        lay.token_stride, lay.head_stride, lay.replica_stride = plan.token_stride, plan.head_stride, 0
        lay.n_tokens, lay.n_heads, lay.n_replicas = n_tokens, heads, 1
        profile.decode_patch_dev_multi(payload.data_ptr(), stride, lay, plan.base_ptr, plan.offsets.data_ptr(),
                                       err.data_ptr(), stream, dst_dtype=plan.dst_dtype)
        return 1
    launches = 0
    for li, pair in enumerate(layers):
        for side, tensor in enumerate(pair):
            if tensor.device != payload.device:
                raise ValueError("cache tensors and payload must be on one device")
            lay = cache_tensor_layout(tensor, n_tokens, pos0)
            profile.decode_patch_dev(payload[li, side].data_ptr(), stride, lay, tensor.data_ptr(),
                                     err.data_ptr(), stream, dst_dtype=dst_dtype_of(tensor))
            launches += 1
    return launches
