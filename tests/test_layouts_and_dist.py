"""Host logic: pkv_layout addressing against NumPy strides, sharding, and the pool
broadcast over a 2-rank gloo group (the CPU stand-in for NCCL)."""
import os
import socket

import numpy as np
import pytest

from provekv_b200 import dist as pdist
from provekv_b200 import pool


def vec_offset(L, batch, v):
    """Python restatement of pkv_vec_offset (provekv_b200/csrc/pkv_common.cuh)."""
    token, head = divmod(v, L.n_heads)
    b2 = batch % L.n_batches[2]
    t = batch // L.n_batches[2]
    b1 = t % L.n_batches[1]
    b0 = t // L.n_batches[1]
    return (L.base + b0 * L.batch_stride[0] + b1 * L.batch_stride[1] + b2 * L.batch_stride[2]
            + token * L.token_stride + head * L.head_stride)


def test_kv_tensor_layout_matches_numpy_indexing():
    shape = pool.KvShape(3, 4, 8)
    A, T, cap, first = 2, 5, 11, 4
    kv = np.arange(A * 3 * 2 * 4 * cap * 8).reshape(A, 3, 2, 4, cap, 8)
    L = pool.kv_tensor_layout(shape, A, T, token_capacity=cap, first_token=first)
    assert L.batch_count == A * 3 * 2 and L.vectors_per_batch == T * 4
    for batch in range(L.batch_count):
        a, rem = divmod(batch, 6)
        layer, side = divmod(rem, 2)
        for v in range(L.vectors_per_batch):
            t, h = divmod(v, 4)  # token-major, head-minor: proveKV/src/pool.rs:246-257
            assert vec_offset(L, batch, v) == kv[a, layer, side, h, first + t, 0]
    with pytest.raises(ValueError):
        pool.kv_tensor_layout(shape, A, T, token_capacity=6, first_token=4)


def test_patch_positions_and_strides():
    # proveKV/scripts/ppl_validate_multi_agent.py:258: pos = n_shared + agent*n_unique + t
    assert pool.agent_patch_position(800, 28, 0) == 800
    assert pool.agent_patch_position(800, 28, 7) == 996
    assert pool.agent_patch_position(800, 28, 7) + 28 == 1024
    assert pool.payload_batch_stride(896, 144) == 896 * 144
    assert pool.payload_batch_stride(3, 12) == 48 and pool.payload_batch_stride(5, 22) == 112
    assert pool.SMOLLM2_1_7B.vectors(1024) == 1_572_864
    assert pool.SMOLLM2_1_7B.vectors(28, 8) == 344_064
    assert pool.LLAMA3_8B.vectors(131072) == 67_108_864


def test_two_tier_plan_addresses_match_numpy_indexing():
    """Every (replica, batch, vector) of the four launches of a rank lands on the element the
    reference's patch loop writes (ppl_validate_multi_agent.py:247-262)."""
    shape = pool.KvShape(4, 2, 8)
    A, ns, nu = 6, 5, 3
    for shard, world in (("agent", 1), ("agent", 2), ("layer", 2), ("agent", 3)):
        seen_prefix_layers, seen_agents = [], []
        for rank in range(world):
            plan = pool.TwoTierPlan(shape, A, ns, nu, world, rank, shard)
            assert plan.cache_tokens == ns + A * nu
            ag, dl, el = plan.agents, plan.dec_layers, plan.enc_layers
            seen_prefix_layers += list(el)
            seen_agents += list(ag)
            cache = np.arange(len(ag) * len(dl) * 2 * 2 * plan.cache_tokens * 8).reshape(
                len(ag), len(dl), 2, 2, plan.cache_tokens, 8)
            assert plan.agent_cache_elems == cache[0].size
            L = plan.prefix_decode_layout()
            assert L.n_replicas == len(ag) and L.batch_count == len(dl) * 2
            for r in range(L.n_replicas):
                for batch in range(L.batch_count):
                    layer, side = divmod(batch, 2)
                    for v in range(L.vectors_per_batch):
                        t, h = divmod(v, 2)
                        assert vec_offset(L, batch, v) + r * L.replica_stride == cache[r, layer, side, h, t, 0]
            L = plan.shell_decode_layout()
            assert L.batch_count == len(ag) * len(dl) * 2 and L.n_replicas == 1
            for batch in range(L.batch_count):
                a, rem = divmod(batch, len(dl) * 2)
                layer, side = divmod(rem, 2)
                for v in range(L.vectors_per_batch):
                    t, h = divmod(v, 2)
                    pos = pool.agent_patch_position(ns, nu, ag[a]) + t
                    assert vec_offset(L, batch, v) == cache[a, layer, side, h, pos, 0]
            src = np.arange(len(el) * 2 * 2 * ns * 8).reshape(len(el), 2, 2, ns, 8)
            L = plan.prefix_encode_layout()
            for batch in range(L.batch_count):
                layer, side = divmod(batch, 2)
                for v in range(L.vectors_per_batch):
                    t, h = divmod(v, 2)
                    assert vec_offset(L, batch, v) == src[layer, side, h, t, 0]
            assert plan.shell_vectors() == len(ag) * len(dl) * 2 * 2 * nu
        assert seen_prefix_layers == list(range(4))
        assert seen_agents == (list(range(A)) if shard == "agent" else list(range(A)) * world)


def test_sharding_covers_everything_once():
    for n, w in [(8, 1), (8, 2), (8, 8), (64, 8), (32, 8), (7, 4), (3, 8)]:
        shards = pdist.all_shards(n, w)
        flat = [i for lo, hi in shards for i in range(lo, hi)]
        assert flat == list(range(n))
        sizes = [hi - lo for lo, hi in shards]
        assert max(sizes) - min(sizes) <= 1
    assert list(pdist.shard_agents(64, 8, 3)) == list(range(24, 32))
    assert list(pdist.shard_layers(32, 8, 7)) == [28, 29, 30, 31]
    with pytest.raises(ValueError):
        pdist.shard_range(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _gloo_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 0 "encodes" the pool; everyone receives the same bytes
        pool_bytes = torch.arange(4096, dtype=torch.int64).to(torch.uint8) if rank == 0 else \
            torch.zeros(4096, dtype=torch.uint8)
        pdist.broadcast_pool(pool_bytes, src=0)
        ok_bcast = bool((pool_bytes == torch.arange(4096, dtype=torch.int64).to(torch.uint8)).all())
        # layer-sharded encode then all-gather
        lo, hi = pdist.shard_range(6, world, rank)
        local = torch.full((hi - lo, 16), rank + 1, dtype=torch.uint8)
        parts = pdist.gather_layer_shards(local, world)
        ok_gather = [int(p[0, 0]) for p in parts] == list(range(1, world + 1))
        # the pool build of the two-tier plan: equal layer blocks gathered into every rank's pool
        plan = pool.TwoTierPlan(pool.KvShape(6, 2, 8), 4, 5, 3, world, rank, "agent")
        mine = torch.tensor([[10 * layer + side] * 16 for layer in plan.enc_layers for side in (0, 1)],
                            dtype=torch.uint8)
        whole = torch.zeros((12, 16), dtype=torch.uint8)
        pdist.all_gather_pool(mine, whole)
        ok_gather = ok_gather and [int(v) for v in whole[:, 0]] == [10 * l + s for l in range(6) for s in (0, 1)]
        agents = list(pdist.shard_agents(8, world, rank))
        slow = pdist.max_over_ranks([1.0 + rank, 5.0 - rank])
        q.put((rank, ok_bcast, ok_gather, agents, slow))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_broadcast_and_sharding():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] and res[1][1] and res[0][2] and res[1][2]
    assert res[0][3] == [0, 1, 2, 3] and res[1][3] == [4, 5, 6, 7]
    assert res[0][4] == [2.0, 5.0] and res[1][4] == [2.0, 5.0]


def test_gpu_numa_cpu_list_from_sysfs(tmp_path):
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    (dev / "numa_node").write_text("1\n")
    (dev / "local_cpulist").write_text("32-35,96,98-99\n")
    assert pdist.gpu_numa_cpus("0000:1B:00.0", str(tmp_path)) == [32, 33, 34, 35, 96, 98, 99]
    (dev / "numa_node").write_text("-1\n")
    assert pdist.gpu_numa_cpus("0000:1b:00.0", str(tmp_path)) == []
    assert pdist.gpu_numa_cpus("0000:ff:00.0", str(tmp_path)) == []


def test_per_vector_wire_framing_round_trips_and_rejects():
    """FB1 (fib-quant/src/codec.rs:81-152) and TQW1 (turbo-quant/src/wire.rs:44-214) framing on the
    host: sizes from the reference's comments (11 + 12 = 23 bytes; 46-byte header), field checks."""
    from provekv_b200 import codec as cd
    rec = bytes(range(12))
    blob = cd.fb1_frame(rec, 5, 16, 2)
    assert len(blob) == 23 and blob[:5] == b"FB1\x01\x05" and blob[5:9] == (16).to_bytes(4, "little")
    assert cd.fb1_parse(blob, 5, 16, 2) == rec
    for bad in (blob[:10], b"XB1" + blob[3:], blob[:3] + b"\x02" + blob[4:], blob + b"\0", blob[:-1]):
        with pytest.raises(cd.DecompressionFailed):
            cd.fb1_parse(bad, 5, 16, 2)
    with pytest.raises(cd.DecompressionFailed):
        cd.fb1_parse(blob, 5, 32, 2)
    trec = bytes(144)
    tb = cd.tqw1_frame(trec, 64, 3, 32, 42, True)
    assert len(tb) == 46 + 144 and tb[:4] == b"TQW1" and tb[8] == 1 and tb[14] == 3
    assert int.from_bytes(tb[38:46], "little") == 144
    assert cd.tqw1_parse(tb, 64, 3, 32, 42, True) == trec
    for bad in (tb[:45], b"TQB1" + tb[4:], tb[:8] + b"\x02" + tb[9:], tb + b"\0"):
        with pytest.raises(cd.DecompressionFailed):
            cd.tqw1_parse(bad, 64, 3, 32, 42, True)
    with pytest.raises(cd.DecompressionFailed):
        cd.tqw1_parse(tb, 64, 3, 32, 43, True)


def test_kv_binary_round_trip_and_layout(tmp_path):
    """The kv binary container of prove_kv_multi_agent_shell.rs:106-122, read the way
    ppl_validate_multi_agent.py:202-224 reads it, and the patch layout of a cache tensor."""
    import json
    import struct

    import torch

    from provekv_b200 import _lib as L
    from provekv_b200 import patch

    rng = np.random.default_rng(3)
    layers = [(rng.standard_normal(48).astype(np.float32), rng.standard_normal(48).astype(np.float32))
              for _ in range(2)]
    manifest = {"num_layers": 2, "num_kv_heads": 2, "head_dim": 8, "num_tokens": 3, "agent_id": "a0"}
    path = tmp_path / "x.kv.bin"
    patch.write_kv_binary(path, manifest, layers)
    raw = path.read_bytes()
    (mlen,) = struct.unpack_from("<Q", raw, 0)
    assert json.loads(raw[8:8 + mlen].decode()) == manifest
    (klen,) = struct.unpack_from("<I", raw, 8 + mlen)
    assert klen == 48 and struct.unpack_from("<48f", raw, 12 + mlen) == tuple(layers[0][0].tolist())
    assert len(raw) == 8 + mlen + 4 * (4 + 4 * 48)
    m, got, nl, nh, hd = patch.read_kv_binary(path)
    assert (m, nl, nh, hd) == (manifest, 2, 2, 8)
    for i in range(2):
        assert np.array_equal(got[i][0], layers[i][0]) and np.array_equal(got[i][1], layers[i][1])
    (tmp_path / "cut.kv.bin").write_bytes(raw[:-5])
    with pytest.raises(ValueError):
        patch.read_kv_binary(tmp_path / "cut.kv.bin")

    cache = torch.zeros((1, 4, 32, 64), dtype=torch.bfloat16)
    lay = patch.cache_tensor_layout(cache, 5, 7)
    assert (lay.base, lay.token_stride, lay.head_stride, lay.n_tokens, lay.n_heads) == (7 * 64, 64, 32 * 64, 5, 4)
    assert patch.dst_dtype_of(cache) == L.DST_BF16 and patch.dst_dtype_of(cache.float()) == L.DST_F32
    with pytest.raises(ValueError):
        patch.cache_tensor_layout(cache, 30, 7)
    with pytest.raises(TypeError):
        patch.dst_dtype_of(cache.to(torch.float64))
    pairs = patch.cache_layers({1: {"k": 3, "v": 4}, 0: {"k": 1, "v": 2}})
    assert pairs == [(1, 2), (3, 4)]


def test_pool_content_addressing_matches_reference_json():
    """Block, layer and pool digests (proveKV/src/codec.rs:83-95, pool.rs:83-103,329-343): blake3 over
    compact JSON with sorted keys, checked against the strings written out by hand."""
    import blake3

    from provekv_b200 import manifest as M

    kb, vb = M.CompressedBlock("fib_k4_n32_batched", b"\x01\x02\x03", 64), M.CompressedBlock("fib_k4_n32_batched", b"", 64)
    assert kb.payload_digest == blake3.blake3(b"\x01\x02\x03").hexdigest() and kb.compressed_bytes == 3
    assert vb.payload_digest == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"  # blake3 of nothing
    assert abs(kb.compression_ratio() - 256 / 3) < 1e-12 and vb.compression_ratio() == 0.0
    layer = M.PoolLayer(5, [kb], [vb])
    text = ('{"key_digests":["%s"],"layer_index":5,"value_digests":["%s"]}' % (kb.payload_digest, vb.payload_digest))
    assert layer.compute_digest() == blake3.blake3(text.encode()).hexdigest()
    shape = M.KvTensorShape("GQA", 24, 32, 32, 64, 2048)
    pid = M.pool_id(["aa", "bb"], "cd", "rd", shape, 42)
    text = ('{"codebook_digest":"cd","layer_digests":["aa","bb"],"rotation_digest":"rd","seed":42,'
            '"shape":{"attention_type":"gqa","head_dim":64,"hidden_size":2048,"num_heads":32,"num_kv_heads":32,'
            '"num_layers":24},"shared_codec":"fib_k4_n32_batched"}')
    assert pid == blake3.blake3(text.encode()).hexdigest()
    assert shape.total_kv_bytes(10) == 24 * 2 * 32 * 64 * 10 * 4
