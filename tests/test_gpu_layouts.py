"""Device-pointer entry points: strided KV tensors, many batches per launch, fused
patch into a larger cache (with replicas), error reporting, the bulk host API, and
the full-size cold-tier configuration checked byte for byte against the oracle."""
import ctypes as C

import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import pool, tables

from kvgen import synthetic_kv

pytestmark = pytest.mark.gpu
SEED = 42


def _torch():
    import torch
    return torch


def _kv_tensor(shape, A, T, seed):
    """kv[agent][layer][side][head][token][dim] and the same vectors in the reference's
    gather order [batch][token][head][dim] (proveKV/src/pool.rs:246-257)."""
    n = A * shape.num_layers * 2 * shape.num_kv_heads * T
    flat = synthetic_kv(n, shape.head_dim, seed=seed)
    kv = flat.reshape(A, shape.num_layers, 2, shape.num_kv_heads, T, shape.head_dim)
    gathered = np.ascontiguousarray(kv.transpose(0, 1, 2, 4, 3, 5)).reshape(
        A * shape.num_layers * 2, T * shape.num_kv_heads, shape.head_dim)
    return kv, gathered


def _profiles(d):
    fib = pk.FibProfile(d, tables.haar_rotation(d, SEED), tables.fib_codebook(d, seed=SEED))
    tq = pk.TurboProfile.from_seed(d, 4, 32, SEED)
    tql = pk.TurboProfile.from_seed(d, 4, 32, SEED, radii_codec=L.RADII_BLOCK_LOG_U8)
    return {"fib": fib, "turbo": tq, "turbo_lossy": tql}


def _oracle_encode(oracle_mod, kind, prof, x):
    if kind == "fib":
        st, p, _, _ = oracle_mod.fib_encode(x, prof.rotation, prof.codebook, nthreads=8)
    else:
        st, p, _, _ = oracle_mod.turbo_encode(x, prof.signs, prof.qjl, bits=4, mode=1,
                                              radii_codec=prof.radii_codec, nthreads=8)
    assert st == 0
    return p


def _oracle_decode(oracle_mod, kind, prof, p, d):
    if kind == "fib":
        st, y, _, _ = oracle_mod.fib_decode(p, d, prof.rotation, prof.codebook, nthreads=8)
    else:
        st, y, _, _ = oracle_mod.turbo_decode(p, d, prof.signs, bits=4, mode=1, projections=32,
                                              radii_codec=prof.radii_codec, nthreads=8)
    assert st == 0
    return y


@pytest.mark.parametrize("kind", ["fib", "turbo", "turbo_lossy"])
@pytest.mark.parametrize("d,heads,T", [(64, 4, 37), (128, 2, 19), (64, 32, 28)])
def test_strided_encode_then_patch_into_cache(oracle_mod, kind, d, heads, T):
    torch = _torch()
    shape = pool.KvShape(3, heads, d)
    A, cap, first, reps = 2, T + 9, 5, 2
    prof = _profiles(d)[kind]
    kv, gathered = _kv_tensor(shape, A, T, seed=d + T)
    n_batches, vpb, rec = A * 3 * 2, T * heads, prof.record_bytes
    kv_dev = torch.from_numpy(kv).cuda()
    stride = pool.payload_batch_stride(vpb, rec)
    payload = torch.zeros((n_batches, stride), dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.encode_dev(kv_dev.data_ptr(), pool.kv_tensor_layout(shape, A, T), payload.data_ptr(), stride,
                    err.data_ptr())
    pk.read_error_word(err.data_ptr())
    got = payload.cpu().numpy()[:, :vpb * rec].reshape(n_batches * vpb, rec)
    want = np.concatenate([_oracle_encode(oracle_mod, kind, prof, gathered[b]) for b in range(n_batches)])
    assert np.array_equal(got, want)

    # decode-and-patch into two replicas of a larger cache at positions [first, first + T)
    cache = torch.full((reps, A, 3, 2, heads, cap, d), 7.0, dtype=torch.float32, device="cuda")
    lay = pool.kv_tensor_layout(shape, A, T, token_capacity=cap, first_token=first, n_replicas=reps,
                                replica_stride=cache.stride(0))
    prof.decode_patch_dev(payload.data_ptr(), stride, lay, cache.data_ptr(), err.data_ptr())
    pk.read_error_word(err.data_ptr())
    dec = _oracle_decode(oracle_mod, kind, prof, want, d).reshape(A, 3, 2, T, heads, d).transpose(0, 1, 2, 4, 3, 5)
    out = cache.cpu().numpy()
    for r in range(reps):
        assert np.array_equal(out[r][..., first:first + T, :].view(np.uint32),
                              np.ascontiguousarray(dec).view(np.uint32))
        assert np.all(out[r][..., :first, :] == 7.0) and np.all(out[r][..., first + T:, :] == 7.0)


@pytest.mark.parametrize("kind", ["fib", "turbo"])
def test_bulk_host_api_equals_per_batch_calls(kind):
    d, n_batches, vpb = 64, 21, 300
    prof = _profiles(d)[kind]
    x = synthetic_kv(n_batches * vpb, d, seed=5).reshape(n_batches, vpb, d)
    hdr = L.FB2_HEADER_BYTES if kind == "fib" else L.TQB1_HEADER_BYTES
    blob = hdr + vpb * prof.record_bytes
    out = np.zeros((n_batches, blob), np.uint8)
    pk.encode_batches_compact(prof, x.ctypes.data, n_batches, vpb, out.ctypes.data, out.size)
    for b in range(n_batches):
        assert out[b].tobytes() == prof.encode_batch_compact(x[b])
    back = np.zeros((n_batches, vpb, d), np.float32)
    pk.decode_batches_compact(prof, out.ctypes.data, n_batches, vpb, back.ctypes.data, back.size)
    for b in range(0, n_batches, 5):
        assert np.array_equal(back[b], prof.decode_batch_compact(out[b].tobytes()))


def test_error_reporting_matches_reference_order(oracle_mod):
    d = 64
    profs = _profiles(d)
    fib, tq = profs["fib"], profs["turbo"]
    x = synthetic_kv(500, d, seed=3)
    x[70, 5] = np.nan
    x[340] = 0.0
    x[10] *= 1e5  # fp16 norm overflow: reported only when no first-pass error exists
    with pytest.raises(L.PkvError) as e:
        fib.encode_batch_compact(x)
    assert (e.value.status, e.value.vector_index) == (L.VEC_NONFINITE_INPUT, 70)
    x[70, 5] = 1.0
    with pytest.raises(L.PkvError) as e:
        fib.encode_batch_compact(x)
    assert (e.value.status, e.value.vector_index) == (L.VEC_ZERO_NORM, 340)
    x[340, 1] = 1.0
    with pytest.raises(L.PkvError) as e:
        fib.encode_batch_compact(x)
    assert (e.value.status, e.value.vector_index) == (L.VEC_NORM_RANGE, 10)
    with pytest.raises(L.PkvError) as e:
        fib.encode_batch_compact(np.zeros((0, d), np.float32))
    assert e.value.status == L.ERR_EMPTY_BATCH

    x = synthetic_kv(400, d, seed=4)
    wire = bytearray(fib.encode_batch_compact(x))
    wire[19 + 12 * 333 + 0] = 0
    wire[19 + 12 * 333 + 1] = 0   # fp16 norm 0
    with pytest.raises(L.PkvError) as e:
        fib.decode_batch_compact(bytes(wire))
    assert (e.value.status, e.value.vector_index) == (L.VEC_BAD_NORM, 333)
    with pytest.raises(L.PkvError) as e:
        fib.decode_batch_compact(bytes(wire[:-1]))
    assert e.value.status == L.ERR_CORRUPT_HEADER
    fib20 = pk.FibProfile(d, fib.rotation, fib.codebook[:20])
    w20 = bytearray(fib20.encode_batch_compact(x))
    w20[19 + 12 * 77 + 2] |= 0x1f
    with pytest.raises(L.PkvError) as e:
        fib20.decode_batch_compact(bytes(w20))
    assert (e.value.status, e.value.vector_index) == (L.VEC_INDEX_RANGE, 77)

    x[222, 63] = -np.inf
    with pytest.raises(L.PkvError) as e:
        tq.encode_batch_compact(x)
    assert (e.value.status, e.value.vector_index) == (L.VEC_NONFINITE_INPUT, 222)
    x[222, 62:] = 3e38
    with pytest.raises(L.PkvError) as e:
        tq.encode_batch_compact(x)
    assert (e.value.status, e.value.vector_index) == (L.VEC_BAD_RADIUS, 222)
    x[222] = 0.0  # zero vectors are fine for turbo (turbo-quant/src/polar.rs:526-533)
    wire = bytearray(tq.encode_batch_compact(x))
    assert np.all(tq.decode_batch_compact(bytes(wire))[222] == 0.0)
    wire[38 + 144 * 9 + 2] = 0xff
    wire[38 + 144 * 9 + 3] = 0xff
    with pytest.raises(L.PkvError) as e:
        tq.decode_batch_compact(bytes(wire))
    assert (e.value.status, e.value.vector_index) == (L.VEC_BAD_RADIUS, 9)
    tql = profs["turbo_lossy"]
    wl = bytearray(tql.encode_batch_compact(x))
    o = 38 + 56 * 100
    wl[o + 32:o + 36], wl[o + 36:o + 40] = wl[o + 36:o + 40], wl[o + 32:o + 36]
    with pytest.raises(L.PkvError) as e:
        tql.decode_batch_compact(bytes(wl))
    assert (e.value.status, e.value.vector_index) == (L.VEC_BAD_RADIUS_RANGE, 100)
    # a lossless profile refuses a lossy payload (byte 15) instead of misreading it
    with pytest.raises(L.PkvError) as e:
        tq.decode_batch_compact(bytes(tql.encode_batch_compact(x)))
    assert e.value.status == L.ERR_CORRUPT_HEADER


def test_adapters_mirror_reference_calls(oracle_mod):
    d = 64
    fib = pk.create_codec(pk.CODEC_FIB_K4_N32_BATCHED, d, fib_config=pk.FibConfig())
    x = synthetic_kv(256, d, seed=11)
    wire = fib.encode_batch_compact(list(x), SEED)
    assert len(wire) == 19 + 256 * 12 and wire[:3] == b"FB2"
    y = fib.decode_batch_compact(wire, SEED)
    prof = fib.build_quantizer(SEED)
    assert np.array_equal(_oracle_encode(oracle_mod, "fib", prof, x).tobytes(), wire[19:])
    assert y.shape == (256, d)
    with pytest.raises(pk.CompressionFailed):
        fib.encode_batch_compact([np.zeros(d, np.float32)] * 5, SEED)
    with pytest.raises(pk.DecompressionFailed):
        fib.decode_batch_compact(b"XX" + wire[2:], SEED)
    for lossy in (False, True):
        tq = pk.TurboQuantAdapter.with_radii_compression(d, 4, 32, lossy)
        w = tq.encode_batch_compact(x, SEED)
        assert len(w) == 38 + 256 * (56 if lossy else 144) and w[15] == int(lossy)
        assert pk.TurboQuantAdapter(d, 4, 32).decode_batch_compact(w, SEED).shape == (256, d)


def test_full_size_cold_tier_bytes_and_roundtrip(oracle_mod):
    """C1: one SmolLM2-1.7B shaped cache, 1024 tokens = 1,572,864 vectors (402.7 MB f32),
    fib k4_n32: every FB2 byte against the multi-threaded oracle, then decode."""
    torch = _torch()
    shape = pool.SMOLLM2_1_7B
    T, d = 1024, 64
    prof = _profiles(d)["fib"]
    n = shape.vectors(T)
    gen = torch.Generator(device="cuda").manual_seed(0)
    scale = torch.exp(0.5 * torch.randn((1, 24, 1, 32, 1, d), generator=gen, device="cuda"))
    kv = (torch.randn((1, 24, 2, 32, T, d), generator=gen, device="cuda") * scale).contiguous()
    vpb, rec = T * 32, prof.record_bytes
    stride = pool.payload_batch_stride(vpb, rec)
    payload = torch.zeros((48, stride), dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.encode_dev(kv.data_ptr(), pool.kv_tensor_layout(shape, 1, T), payload.data_ptr(), stride,
                    err.data_ptr())
    pk.read_error_word(err.data_ptr())
    got = payload.cpu().numpy().reshape(n, rec)
    assert 48 * 19 + got.size == 18_875_280  # results/ppl/smollm2-1.7b/.../state.json:53
    gathered = kv.permute(0, 1, 2, 4, 3, 5).reshape(n, d).cpu().numpy()
    want = _oracle_encode(oracle_mod, "fib", prof, gathered)
    assert np.array_equal(got, want)
    out = torch.zeros_like(kv)
    prof.decode_patch_dev(payload.data_ptr(), stride, pool.kv_tensor_layout(shape, 1, T), out.data_ptr(),
                          err.data_ptr())
    pk.read_error_word(err.data_ptr())
    sample = slice(0, n, 37)
    dec = out.permute(0, 1, 2, 4, 3, 5).reshape(n, d)[sample].cpu().numpy()
    ref = _oracle_decode(oracle_mod, "fib", prof, want[sample], d)
    assert np.array_equal(dec.view(np.uint32), ref.view(np.uint32))
    rel = float(((out - kv) ** 2).sum() / (kv ** 2).sum())
    assert 0.05 < rel < 0.4


@pytest.mark.parametrize("kind", ["turbo", "turbo_lossy"])
def test_full_size_hot_shells_bytes_and_roundtrip(oracle_mod, kind):
    """C2: 8 agents x 28-token hot shells of a SmolLM2-1.7B shaped cache = 344,064 vectors
    (88.1 MB f32), turbo b=4: every TQB1 record byte against the multi-threaded oracle (11 M QJL
    signs, so all three tiers of the sign certification are taken many times), then the decode
    patched into an 800-token cache at each agent's position."""
    torch = _torch()
    shape = pool.SMOLLM2_1_7B
    A, T, d, cap = 8, 28, 64, 1024
    prof = _profiles(d)[kind]
    n = A * shape.vectors(T)
    gen = torch.Generator(device="cuda").manual_seed(1)
    scale = torch.exp(0.5 * torch.randn((1, 24, 1, 32, 1, d), generator=gen, device="cuda"))
    kv = (torch.randn((A, 24, 2, 32, T, d), generator=gen, device="cuda") * scale).contiguous()
    vpb, rec = T * 32, prof.record_bytes
    stride = pool.payload_batch_stride(vpb, rec)
    payload = torch.zeros((A * 48, stride), dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.encode_dev(kv.data_ptr(), pool.kv_tensor_layout(shape, A, T), payload.data_ptr(), stride,
                    err.data_ptr())
    pk.read_error_word(err.data_ptr())
    got = payload[:, :vpb * rec].cpu().numpy().reshape(n, rec)
    gathered = kv.permute(0, 1, 2, 4, 3, 5).reshape(n, d).cpu().numpy()
    want = _oracle_encode(oracle_mod, kind, prof, gathered)
    assert np.array_equal(got, want)
    first = pool.agent_patch_position(800, T, 0)
    cache = torch.full((A, 24, 2, 32, cap, d), 7.0, device="cuda")
    prof.decode_patch_dev(payload.data_ptr(), stride,
                          pool.kv_tensor_layout(shape, A, T, token_capacity=cap, first_token=first),
                          cache.data_ptr(), err.data_ptr())
    pk.read_error_word(err.data_ptr())
    patched = cache[:, :, :, :, first:first + T, :]
    sample = slice(0, n, 53)
    dec = patched.permute(0, 1, 2, 4, 3, 5).reshape(n, d)[sample].cpu().numpy()
    ref = _oracle_decode(oracle_mod, kind, prof, want[sample], d)
    assert np.array_equal(dec.view(np.uint32), ref.view(np.uint32))
    assert bool((cache[:, :, :, :, :first, :] == 7.0).all()) and bool((cache[:, :, :, :, first + T:, :] == 7.0).all())
    rel = float(((patched - kv) ** 2).sum() / (kv ** 2).sum())
    assert 0.01 < rel < 0.4


@pytest.mark.parametrize("codec", ["fib", "turbo"])
def test_scaled_long_context_d128_bytes_and_decode(oracle_mod, codec):
    """C5 scaled (d=128, 8 KV heads, bf16-valued inputs with 1 % outlier channels x 20): 2 M vectors,
    every record byte and a 200k-vector sample of the decode against the oracle.  The 67 M QJL signs
    of the turbo case include dots within 1e-8 of zero relative to their terms, which only come out
    right if the residual is bit-exact."""
    import parity_report
    shape = pool.LLAMA3_8B
    if codec == "fib":
        bad = parity_report.run(_torch(), "C5", "fib d=128 scaled", shape, 1, 4096, "fib", seed=6, outliers=True)
    else:
        bad = parity_report.run(_torch(), "C5", "turbo d=128 scaled", shape, 16, 256, "turbo", seed=7, outliers=True)
    assert bad == 0


def test_per_vector_payloads_fb1_and_tqw1(oracle_mod):
    """KVecCodec::{encode, encode_batch, decode, decode_batch} (proveKV/src/codec.rs:341-412,581-667):
    the per-vector FB1 / TQW1 payloads carry the same records as the batched formats -- single-vector
    numerics for fib `encode`, batch numerics for `encode_batch`."""
    from provekv_b200 import codec as cd
    d = 64
    x = synthetic_kv(40, d, seed=21)
    fib = pk.create_codec(pk.CODEC_FIB_K4_N32, d, fib_config=pk.FibConfig())
    prof = fib.build_quantizer(SEED)
    blobs = fib.encode_batch(list(x), SEED)
    st, want, _, _ = oracle_mod.fib_encode(x, prof.rotation, prof.codebook, numerics=L.FIB_NUMERICS_BATCH)
    assert st == 0 and len(blobs) == 40 and all(len(b) == 23 for b in blobs)
    assert b"".join(b[11:] for b in blobs) == want.tobytes()
    one = fib.encode(x[7], SEED)
    st, w1, _, _ = oracle_mod.fib_encode(x[7:8], prof.rotation, prof.codebook, numerics=L.FIB_NUMERICS_SINGLE)
    assert st == 0 and one == cd.fb1_frame(w1.tobytes(), 5, 16, 2)
    y = fib.decode_batch(blobs, SEED)
    st, ref, _, _ = oracle_mod.fib_decode(want, d, prof.rotation, prof.codebook)
    assert np.array_equal(y.view(np.uint32), ref.view(np.uint32))
    # KVecCodec::decode of one payload: FibQuantizer::decode, binary64 inverse rotation
    st, ex, _, _ = oracle_mod.fib_decode_exact(want, d, prof.rotation, prof.codebook)
    assert st == 0
    for i in (0, 7, 39):
        assert np.array_equal(fib.decode(blobs[i], SEED).view(np.uint32), ex[i].view(np.uint32))
    assert np.array_equal(prof.decode_exact(want.tobytes()).view(np.uint32), ex.view(np.uint32))
    assert np.abs(ex - ref).max() < 1e-4 and not np.array_equal(ex, ref)  # decode_batch_fast_parity.rs:37-47
    bad = bytearray(want[3].tobytes())
    bad[2] |= 0x1f  # index 31 of a 32-entry codebook is fine; shrink the codebook to make it out of range
    small = pk.FibProfile(d, prof.rotation, prof.codebook[:17])
    with pytest.raises(L.PkvError) as ei:
        small.decode_exact(bytes(bad))
    assert ei.value.status == L.VEC_INDEX_RANGE
    with pytest.raises(pk.DecompressionFailed):
        fib.decode_batch([blobs[0][:-1]], SEED)

    tq = pk.create_codec(pk.CODEC_TURBO_8BIT, d, turbo_config=pk.TurboConfig(bits=4, projections=32))
    tprof = tq.build_quantizer(SEED)
    tb = tq.encode_batch(list(x), SEED)
    st, twant, _, _ = oracle_mod.turbo_encode(x, tprof.signs, tprof.qjl, bits=4, mode=1, radii_codec=0)
    assert st == 0 and all(len(b) == 46 + 144 and b[:4] == b"TQW1" for b in tb)
    assert b"".join(b[46:] for b in tb) == twant.tobytes()
    assert tq.encode(x[3], SEED) == tb[3]
    ty = tq.decode_batch(tb, SEED)
    st, tref, _, _ = oracle_mod.turbo_decode(twant, d, tprof.signs, bits=4, mode=1, projections=32, radii_codec=0)
    assert np.array_equal(ty.view(np.uint32), tref.view(np.uint32))
    assert np.array_equal(tq.decode(tb[5], SEED), ty[5])
    with pytest.raises(pk.DecompressionFailed):
        tq.decode(tb[0][:4] + b"\x02" + tb[0][5:], SEED)
