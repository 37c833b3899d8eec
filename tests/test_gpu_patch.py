"""Decode-and-patch into a framework's per-layer caches: fp16 / bf16 / f32 cache tensors, one
allocation per (layer, K|V) as in a transformers DynamicCache, replicas, and the value flow
kv-binary file -> cache of proveKV/scripts/ppl_validate_multi_agent.py:202-293."""
import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import patch, pool

from kvgen import synthetic_kv
from test_gpu_layouts import _oracle_decode, _oracle_encode, _profiles

pytestmark = pytest.mark.gpu


def _bits16(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy()


def _reference_patch(torch, dec, layers, heads, T, d, dtype, caps, pos0, fill):
    """patch_cache_with_multi_agent_kv, ppl_validate_multi_agent.py:247-262: per token,
    `k[0, :, pos, :] = torch.tensor(flat[t*stride:(t+1)*stride], dtype=k.dtype).view(H, d)`."""
    out = []
    for li in range(layers):
        pair = []
        for side in range(2):
            c = torch.full((1, heads, caps[li], d), fill, dtype=dtype)
            flat = dec[li, side].reshape(T, heads * d)
            for t in range(T):
                c[0, :, pos0 + t, :] = torch.tensor(flat[t].tolist(), dtype=dtype).view(heads, d)
            pair.append(c)
        out.append(pair)
    return out


@pytest.mark.parametrize("kind", ["fib", "turbo", "turbo_lossy"])
@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("d,heads,T,alike", [(64, 4, 21, True), (128, 2, 9, True), (64, 4, 21, False)])
def test_patch_per_layer_caches_of_every_dtype(oracle_mod, kind, dtype_name, d, heads, T, alike):
    import torch
    dtype = getattr(torch, dtype_name)
    layers, cap, pos0 = 3, T + 11, 6
    prof = _profiles(d)[kind]
    vpb, rec = T * heads, prof.record_bytes
    x = synthetic_kv(layers * 2 * vpb, d, seed=d + T).reshape(layers * 2, vpb, d)
    if dtype_name == "float16" and kind != "fib":  # (a fib norm that large does not fit its fp16 field)
        x[0, 0, :] *= 3.0e4  # decoded values beyond the fp16 range must become infinities
    stride = pool.payload_batch_stride(vpb, rec)
    want = [_oracle_encode(oracle_mod, kind, prof, x[b]) for b in range(layers * 2)]
    host = np.zeros((layers, 2, stride), np.uint8)
    for b, p in enumerate(want):
        host[b // 2, b % 2, :vpb * rec] = p.reshape(-1)
    payload = torch.from_numpy(host).cuda()
    dec = np.stack([_oracle_decode(oracle_mod, kind, prof, p, d) for p in want]).reshape(layers, 2, T, heads, d)

    # alike tensors take one launch for the whole cache; layers of different capacity one per tensor
    caps = [cap if alike else cap + li for li in range(layers)]
    try:  # the reference installs the tensors in a DynamicCache (ppl_validate_multi_agent.py:282-293)
        from transformers import DynamicCache, DynamicLayer
        cache = DynamicCache()
        while len(cache.layers) < layers:
            cache.layers.append(DynamicLayer())
        for li, layer in enumerate(cache.layers):
            layer.keys = torch.full((1, heads, caps[li], d), 7.0, dtype=dtype, device="cuda")
            layer.values = torch.full((1, heads, caps[li], d), 7.0, dtype=dtype, device="cuda")
    except Exception:
        cache = [(torch.full((1, heads, caps[li], d), 7.0, dtype=dtype, device="cuda"),
                  torch.full((1, heads, caps[li], d), 7.0, dtype=dtype, device="cuda")) for li in range(layers)]
    assert (patch.plan_cache(cache) is not None) == alike

    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    before = L.lib().pkv_launch_count()
    n = patch.patch_cache(prof, payload, cache, T, pos0, err)
    pk.read_error_word(err.data_ptr())
    assert n == (1 if alike else 2 * layers) and L.lib().pkv_launch_count() - before == n

    ref = _reference_patch(torch, dec, layers, heads, T, d, dtype, caps, pos0, 7.0)
    for li, (k, v) in enumerate(patch.cache_layers(cache)):
        for side, got in enumerate((k, v)):
            exp = ref[li][side]
            if dtype == torch.float32:
                assert np.array_equal(got.cpu().numpy().view(np.uint32), exp.numpy().view(np.uint32))
            else:
                assert np.array_equal(_bits16(got), _bits16(exp)), (kind, dtype_name, li, side)
    if dtype_name == "float16" and kind != "fib":
        assert torch.isinf(patch.cache_layers(cache)[0][0][0, :, pos0, :].float()).any()


@pytest.mark.parametrize("kind", ["fib", "turbo"])
def test_half_precision_replicas_and_alignment_rule(oracle_mod, kind):
    import torch
    d, heads, T, reps, cap = 64, 8, 13, 3, 16
    prof = _profiles(d)[kind]
    vpb, rec = T * heads, prof.record_bytes
    x = synthetic_kv(vpb, d, seed=5)
    p = _oracle_encode(oracle_mod, kind, prof, x)
    stride = pool.payload_batch_stride(vpb, rec)
    host = np.zeros(stride, np.uint8)
    host[:vpb * rec] = p.reshape(-1)
    payload = torch.from_numpy(host).cuda()
    dec = torch.from_numpy(_oracle_decode(oracle_mod, kind, prof, p, d).reshape(T, heads, d)).to(torch.bfloat16)
    caches = torch.zeros((reps, heads, cap, d), dtype=torch.bfloat16, device="cuda")
    lay = patch.cache_tensor_layout(caches[0], T, 2)
    lay.n_replicas, lay.replica_stride = reps, caches.stride(0)
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.decode_patch_dev(payload.data_ptr(), stride, lay, caches.data_ptr(), err.data_ptr(),
                          dst_dtype=L.DST_BF16)
    pk.read_error_word(err.data_ptr())
    for r in range(reps):
        assert np.array_equal(_bits16(caches[r, :, 2:2 + T, :]), _bits16(dec.permute(1, 0, 2)))
        assert float(caches[r, :, :2, :].abs().max()) == 0.0 and float(caches[r, :, 2 + T:, :].abs().max()) == 0.0
    # 16-bit caches need offsets in multiples of 8 elements; an unknown type code is refused
    lay.base += 4
    with pytest.raises(pk.PkvError):
        prof.decode_patch_dev(payload.data_ptr(), stride, lay, caches.data_ptr(), err.data_ptr(),
                              dst_dtype=L.DST_BF16)
    lay.base -= 4
    with pytest.raises(pk.PkvError):
        prof.decode_patch_dev(payload.data_ptr(), stride, lay, caches.data_ptr(), err.data_ptr(), dst_dtype=3)


def test_kv_binary_file_to_cache(oracle_mod, tmp_path):
    """encode on the GPU -> decode to the flat [token][head][dim] lists the reference writes to a
    kv binary file -> read it back -> the values a cache patched from that file would hold equal
    the cache patched by the fused kernel."""
    import torch
    d, heads, T, layers = 64, 4, 12, 2
    prof = _profiles(d)["turbo"]
    x = synthetic_kv(layers * 2 * T * heads, d, seed=77).reshape(layers * 2, T * heads, d)
    blobs = [prof.encode_batch_compact(x[b]) for b in range(layers * 2)]
    flat = [prof.decode_batch_compact(b).reshape(-1) for b in blobs]
    path = tmp_path / "agent.kv.bin"
    patch.write_kv_binary(path, {"num_layers": layers, "num_kv_heads": heads, "head_dim": d, "num_tokens": T},
                          [(flat[2 * i], flat[2 * i + 1]) for i in range(layers)])
    manifest, from_file, nl, nh, hd = patch.read_kv_binary(path)
    assert (nl, nh, hd, manifest["num_tokens"]) == (layers, heads, d, T)

    rec, vpb = prof.record_bytes, T * heads
    stride = pool.payload_batch_stride(vpb, rec)
    host = np.zeros((layers, 2, stride), np.uint8)
    for b, blob in enumerate(blobs):
        host[b // 2, b % 2, :vpb * rec] = np.frombuffer(blob, np.uint8)[L.TQB1_HEADER_BYTES:]
    cache = {i: {"k": torch.zeros((1, heads, T, d), dtype=torch.float16, device="cuda"),
                 "v": torch.zeros((1, heads, T, d), dtype=torch.float16, device="cuda")} for i in range(layers)}
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    patch.patch_cache(prof, torch.from_numpy(host).cuda(), cache, T, 0, err)
    pk.read_error_word(err.data_ptr())
    for i in range(layers):
        for side, name in enumerate("kv"):
            exp = torch.from_numpy(from_file[i][side].reshape(T, heads, d)).to(torch.float16).permute(1, 0, 2)
            assert np.array_equal(_bits16(cache[i][name][0]), _bits16(exp))


@pytest.mark.parametrize("kind", ["fib", "turbo"])
def test_multi_tensor_launch_checks_offsets_on_the_device(oracle_mod, kind):
    """A tensor offset that is not a multiple of 16 bytes is reported (PKV_VEC_MISALIGNED_DST, with
    the batch's first vector) and that batch is skipped; the other batches are written."""
    import torch
    d, heads, T, nb = 64, 4, 8, 3
    prof = _profiles(d)[kind]
    vpb, rec = T * heads, prof.record_bytes
    x = synthetic_kv(nb * vpb, d, seed=9).reshape(nb, vpb, d)
    stride = pool.payload_batch_stride(vpb, rec)
    host = np.zeros((nb, stride), np.uint8)
    want = [_oracle_encode(oracle_mod, kind, prof, x[b]) for b in range(nb)]
    for b in range(nb):
        host[b, :vpb * rec] = want[b].reshape(-1)
    payload = torch.from_numpy(host).cuda()
    arena = torch.zeros(nb * heads * T * d + 64, dtype=torch.float32, device="cuda")
    per = heads * T * d
    lay = patch.cache_tensor_layout(arena[:per].view(heads, T, d), T, 0)
    lay.n_batches[0] = nb
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    for bad in (None, 1):
        arena.zero_()
        err.fill_(-1)
        offs = [b * per for b in range(nb)]
        if bad is not None:
            offs[bad] += 2
        table = torch.tensor(offs, dtype=torch.int64, device="cuda")
        prof.decode_patch_dev_multi(payload.data_ptr(), stride, lay, arena.data_ptr(), table.data_ptr(),
                                    err.data_ptr())
        if bad is None:
            pk.read_error_word(err.data_ptr())
        else:
            with pytest.raises(pk.PkvError) as e:
                pk.read_error_word(err.data_ptr())
            assert e.value.status == L.VEC_MISALIGNED_DST and e.value.vector_index == bad * vpb
        out = arena.cpu().numpy()
        for b in range(nb):
            got = out[b * per:(b + 1) * per].reshape(heads, T, d)
            if b == bad:
                assert not out[b * per:(b + 1) * per].any()
            else:
                exp = _oracle_decode(oracle_mod, kind, prof, want[b], d).reshape(T, heads, d).transpose(1, 0, 2)
                assert np.array_equal(got.view(np.uint32), np.ascontiguousarray(exp).view(np.uint32))


def test_shared_pool_built_on_the_gpu_from_the_reference_corpus_layout(oracle_mod):
    """build_shared_pool encodes every (layer, K|V) batch of a [token][layer][head][K|V][dim] corpus
    in one launch; the blobs must equal the per-batch encode_batch_compact results of
    proveKV/src/pool.rs:246-266 and the digests must chain as in pool.rs:83-103,329-343."""
    from provekv_b200 import manifest as M
    d, H, Lc, T = 64, 4, 3, 37
    prof = _profiles(d)["fib"]
    corpus = synthetic_kv(T * Lc * H * 2, d, seed=21).reshape(T, Lc * H * 2 * d)
    shape = M.KvTensorShape("mha", Lc, H, H, d, H * d)
    before = L.lib().pkv_launch_count()
    pool_ = M.build_shared_pool(prof, corpus, shape, 42, "cb-digest", "rot-digest")
    assert L.lib().pkv_launch_count() - before == 2  # the encoder and its exact fix-up pass
    x = corpus.reshape(T, Lc, H, 2, d)
    for li, layer in enumerate(pool_["layers"]):
        for side, block in enumerate((layer.key_blocks[0], layer.value_blocks[0])):
            vectors = np.ascontiguousarray(x[:, li, :, side, :]).reshape(T * H, d)  # token-major, head-minor
            want = oracle_mod.fb2_header(d, T * H) + _oracle_encode(oracle_mod, "fib", prof, vectors).tobytes()
            assert block.encoded_payload == want and block.original_dim == d
        assert layer.block_digest == layer.compute_digest() == pool_["layer_digests"][li]
    assert pool_["pool_id"] == M.pool_id(pool_["layer_digests"], "cb-digest", "rot-digest", shape, 42)
    assert pool_["pool_size_bytes"] == Lc * 2 * (19 + T * H * 12) and pool_["raw_size_bytes"] == corpus.size * 4
    manifest, receipt = pool_["manifest"], pool_["receipt"]
    manifest.validate()
    receipt.validate()
    assert receipt.backend == "gpu" and receipt.pool_digest == manifest.pool_id == pool_["pool_id"]
    assert receipt.layer_digests == pool_["layer_digests"] and receipt.total_tokens == manifest.num_shared_tokens == T
    assert manifest.compression_ratio == receipt.compression_ratio == corpus.size * 4 / pool_["pool_size_bytes"]
    assert manifest.shared_codec == "fib_k4_n32_batched" and manifest.build_seed == receipt.seeded_with == 42


@pytest.mark.parametrize("lossy", [False, True])
def test_shell_materialised_on_the_gpu_and_the_injection_trace(oracle_mod, lossy):
    """materialize_shell encodes an agent's own tokens as one TQB1 blob per (layer, K|V)
    (proveKV/src/shell.rs:232-296): the blobs equal the oracle's encode of the same gathers, the layer and
    shell digests chain as in shell.rs:48-67,322-337, the manifest's codec id follows the policy, and an
    agent with no tokens of its own gets the empty shell of shell.rs:156-196."""
    from provekv_b200 import manifest as M
    from provekv_b200 import records as R
    d, H, Lc, T, seed = 64, 2, 3, 23, 42
    shape = M.KvTensorShape("gqa", Lc, 8, H, d, 8 * d)
    policy = R.CompressionPolicy.default_two_tier_lossy() if lossy else R.CompressionPolicy.default_two_tier()
    pm = R.PoolManifest.new("pool-id", shape, policy, 800, Lc, 1000, 100000, seed, 11)
    prof = _profiles(d)["turbo_lossy" if lossy else "turbo"]
    tokens = synthetic_kv(T * Lc * H * 2, d, seed=33).reshape(T, Lc * H * 2 * d)
    shell, receipt = M.materialize_shell(pm, "agent_3", tokens, seed, profile=prof, materialized_at_unix=12)
    codec = "turbo_4bit_batched_lossy" if lossy else "turbo_4bit_batched"
    x = tokens.reshape(T, Lc, H, 2, d)
    header = oracle_mod.tqb1_header(d, 4, 1, 32, prof.radii_codec, prof.seed, T * H)
    total = 0
    for li, layer in enumerate(shell.unique_layers):
        for side, block in enumerate((layer.key_blocks[0], layer.value_blocks[0])):
            vectors = np.ascontiguousarray(x[:, li, :, side, :]).reshape(T * H, d)
            want = header + _oracle_encode(oracle_mod, "turbo", prof, vectors).tobytes()
            assert block.encoded_payload == want and block.codec == codec and block.original_dim == d
            total += len(want)
        assert layer.layer_index == li and layer.block_digest == layer.compute_digest()
    sm = shell.shell_manifest
    sm.validate()
    receipt.validate()
    assert (sm.shell_codec, sm.num_unique_tokens, sm.num_unique_layers, sm.shell_size_bytes) == (codec, T, Lc, total)
    assert sm.component_kinds == ["KeyValue"] * Lc and sm.pool_digest == shell.pool_digest == "pool-id"
    assert (sm.materialize_seed, sm.materialized_at_unix, sm.head_dim, sm.num_kv_heads) == (seed, 12, d, H)
    assert receipt.shell_digest == M.shell_digest("agent_3", "pool-id", [l.block_digest for l in shell.unique_layers], seed)
    assert receipt.shell_size_bytes == total and receipt.num_unique_tokens == T
    trace = M.injection_receipt("agent_3", pm, ["p0", "p1", "p2"], shell, receipt.shell_digest, 13)
    assert trace.blocks_injected == 2 * Lc and trace.block_traces[1].target_position == 800
    empty, r0 = M.materialize_shell(pm, "agent_4", np.zeros((0, Lc * H * 2 * d), np.float32), seed)
    assert empty.unique_layers == [] and r0.shell_size_bytes == 0 and empty.shell_manifest.num_unique_layers == Lc
    assert r0.shell_digest == M.shell_digest("agent_4", "pool-id", [], seed)
    bad = tokens.copy()
    bad[5, 17] = np.inf
    with pytest.raises(pk.codec.CorruptPayload, match="agent token 5 contains non-finite values"):
        M.materialize_shell(pm, "agent_3", bad, seed, profile=prof)
    with pytest.raises(pk.codec.DimensionMismatch):
        M.materialize_shell(pm, "agent_3", tokens[:, :-1], seed, profile=prof)
