"""The oracle against every fact the reference's own tests state for this path.

The reference holds no known-answer vectors for codes or tables, so these are the
pins that exist: byte sizes, header offsets, bit order, tie rule, impulse response,
batch == single decode, fast-vs-f64 decode tolerance.  Each test names its source.
"""
import ctypes as C
import struct

import numpy as np
import pytest

from provekv_b200 import tables


def _lcg_data(seed, k, n_codewords):
    """gpu-backend/src/simd_nearest.rs:125-147 (make_test_data)."""
    s = seed
    vals = []
    for _ in range(n_codewords * k + k):
        s = (s * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
        v = s >> 32
        if v >= 1 << 31:
            v -= 1 << 32
        vals.append(np.float32(np.float32(v) / np.float32(2147483647)) * np.float32(0.5))
    a = np.array(vals, np.float32)
    return a[n_codewords * k:], a[:n_codewords * k]


def test_fb2_size_formula(oracle_mod):
    # fib-quant/src/codec.rs:1126-1127: 16 vectors at d=64 -> 19 + 16*12 = 211 bytes
    assert oracle_mod.fib_record_bytes(64) == 12
    assert 19 + 16 * oracle_mod.fib_record_bytes(64) == 211
    assert oracle_mod.fib_record_bytes(128) == 22
    # receipts re-derived from CLAIMS.json / results/ppl/.../state.json:53
    assert 1_228_800 * 12 + 48 * 19 == 14_746_512
    assert 1_572_864 * 12 + 48 * 19 == 18_875_280


def test_tqb1_size_formulas(oracle_mod):
    # CLAIMS.json shell_bytes_per_agent: 43,008 vectors x 144 B + 48 x 38 B; lossy 56 B
    assert oracle_mod.turbo_record_bytes(64, 4, 1, 32, 0) == 144
    assert oracle_mod.turbo_record_bytes(64, 4, 1, 32, 1) == 56
    assert 43_008 * 144 + 48 * 38 == 6_194_976
    assert 43_008 * 56 + 48 * 38 == 2_410_272
    # results/ppl_shell/.../shell_roundtrip_lossless.receipt.json:6 (b=8, 224 tokens)
    assert oracle_mod.turbo_record_bytes(64, 8, 1, 32, 0) == 160
    assert 344_064 * 160 + 48 * 38 == 55_052_064
    assert oracle_mod.turbo_record_bytes(128, 4, 1, 32, 0) == 284
    assert oracle_mod.turbo_record_bytes(128, 4, 1, 32, 1) == 100


def test_bit_order_lsb_first(oracle_mod):
    # gpu-backend/src/fallback.rs:389-397: [0,1,2,3] at 2 bits -> 0b11100100
    vals = np.array([0, 1, 2, 3], np.uint32)
    out = np.zeros(1, np.uint8)
    oracle_mod.lib().pkvo_pack_bits(vals.ctypes.data_as(C.c_void_p), 4, 2, out.ctypes.data_as(C.c_void_p))
    assert out[0] == 0b11100100


@pytest.mark.parametrize("width", [1, 3, 5, 7, 11])
def test_bitpack_roundtrip_and_padding(oracle_mod, width):
    # fib-quant/tests/{bitpack_indices,property_bitpack}.rs, turbo-quant/tests/bitpack.rs
    rng = np.random.default_rng(width)
    count = 13
    vals = rng.integers(0, 1 << width, count).astype(np.uint32)
    nbytes = (count * width + 7) // 8
    buf = np.zeros(nbytes, np.uint8)
    lib = oracle_mod.lib()
    lib.pkvo_pack_bits(vals.ctypes.data_as(C.c_void_p), count, width, buf.ctypes.data_as(C.c_void_p))
    back = np.zeros(count, np.uint32)
    assert lib.pkvo_unpack_bits(buf.ctypes.data_as(C.c_void_p), count, width,
                                back.ctypes.data_as(C.c_void_p)) == 1
    assert np.array_equal(vals, back)
    if (count * width) % 8:
        buf[-1] |= 0x80  # a non-zero padding bit must be rejected
        assert lib.pkvo_unpack_bits(buf.ctypes.data_as(C.c_void_p), count, width,
                                    back.ctypes.data_as(C.c_void_p)) == 0


def _nearest(oracle_mod, sample, cb, k, order):
    s = np.ascontiguousarray(sample, np.float32)
    c = np.ascontiguousarray(cb, np.float32)
    return oracle_mod.lib().pkvo_nearest_codeword(s.ctypes.data_as(C.c_void_p), c.ctypes.data_as(C.c_void_p),
                                                  c.size // k, k, order)


def test_argmin_simd_matches_scalar_on_lcg_seeds(oracle_mod):
    # gpu-backend/src/simd_nearest.rs:150-158
    for seed in range(16):
        sample, cb = _lcg_data(seed, 4, 32)
        assert _nearest(oracle_mod, sample, cb, 4, 0) == _nearest(oracle_mod, sample, cb, 4, 1)


def test_argmin_exact_codeword(oracle_mod):
    # gpu-backend/src/simd_nearest.rs:161-167
    cb = (np.arange(32 * 4, dtype=np.float32) * np.float32(0.01)).astype(np.float32)
    for order in (0, 1):
        assert _nearest(oracle_mod, cb[20:24], cb, 4, order) == 5


def test_argmin_k2_fallback_and_tie_goes_to_lowest_index(oracle_mod):
    # simd_nearest.rs:170-176 and gpu-backend/src/fallback.rs:433-443
    cb = np.array([0, 0, 1, 1, 2, 2, 3, 3], np.float32)
    assert _nearest(oracle_mod, np.array([0.1, 0.1], np.float32), cb, 2, 0) == 0
    tie = np.zeros((32, 4), np.float32)
    tie[:] = 5.0
    tie[8] = tie[16] = [1, 0, 0, 0]
    for order in (0, 1):
        assert _nearest(oracle_mod, np.zeros(4, np.float32), tie, 4, order) == 8


def test_hadamard_unit_impulse(oracle_mod):
    # gpu-backend/src/fallback.rs:312-335: impulse -> +-1/sqrt(d) everywhere
    for d in (64, 128):
        v = np.zeros(d, np.float32)
        v[3] = 1.0
        oracle_mod.lib().pkvo_fwht_normalized(v.ctypes.data_as(C.c_void_p), d)
        assert np.allclose(np.abs(v), 1.0 / np.sqrt(d), rtol=0, atol=1e-7)
        # second application restores the impulse (H/sqrt(d) is an involution)
        oracle_mod.lib().pkvo_fwht_normalized(v.ctypes.data_as(C.c_void_p), d)
        want = np.zeros(d, np.float32)
        want[3] = 1.0
        assert np.allclose(v, want, atol=1e-6)


def test_fb2_header_fields(oracle_mod):
    # layout comment fib-quant/src/codec.rs:195-220
    h = oracle_mod.fb2_header(64, 1000)
    assert h[:3] == b"FB2" and h[3] == 1 and h[4] == 5 and h[5] == 0
    assert struct.unpack_from("<I", h, 6)[0] == 16
    assert struct.unpack_from("<I", h, 10)[0] == 1000
    assert h[14] == 0
    assert struct.unpack_from("<HH", h, 15) == (2, 10)
    assert oracle_mod.fb2_parse(h + bytes(12 * 1000), 64) == (0, 1000)
    assert oracle_mod.fb2_parse(h + bytes(12 * 999), 64)[0] != 0          # truncated
    assert oracle_mod.fb2_parse(b"FB1" + h[3:] + bytes(12000), 64)[0] != 0  # magic
    assert oracle_mod.fb2_parse(h + bytes(12 * 1000), 128)[0] != 0        # profile mismatch


def test_tqb1_header_offsets(oracle_mod):
    # turbo-quant/tests/wire_format.rs:3-7, wire.rs:276-290, byte 15 flag wire.rs:979-983
    h = oracle_mod.tqb1_header(64, 4, 1, 32, 1, 42, 7)
    assert len(h) == 38 and h[:4] == b"TQB1"
    assert struct.unpack_from("<HH", h, 4) == (1, 1)
    assert h[8] == 2 and h[9] == 0
    assert struct.unpack_from("<I", h, 10)[0] == 64
    assert h[14] == 3 and h[15] == 1 and h[16:18] == b"\0\0"
    assert struct.unpack_from("<I", h, 18)[0] == 32
    assert struct.unpack_from("<Q", h, 22)[0] == 42
    assert struct.unpack_from("<II", h, 30) == (7, 56)
    assert oracle_mod.tqb1_header(64, 4, 1, 32, 0, 42, 7)[15] == 0
    ok = h + bytes(56 * 7)
    assert oracle_mod.tqb1_parse(ok, 64, 4, 1, 32, 42) == (0, 7, 1)
    assert oracle_mod.tqb1_parse(ok + b"\0", 64, 4, 1, 32, 42)[0] != 0  # trailing byte
    assert oracle_mod.tqb1_parse(ok, 64, 4, 1, 32, 43)[0] != 0          # seed mismatch
    assert oracle_mod.tqb1_parse(ok, 64, 8, 1, 32, 42)[0] != 0          # polar bits mismatch


def _sin_vectors(n, d):
    # the deterministic inputs of fib-quant/src/codec.rs:1099-1105
    i = np.arange(n)[:, None]
    j = np.arange(d)[None, :]
    return np.sin((i * d + j) * 0.013).astype(np.float32)


def test_fib_fast_decode_within_1e4_of_f64_decode(oracle_mod):
    # fib-quant/tests/decode_batch_fast_parity.rs:37-47
    d = 64
    rot, cb = tables.haar_rotation(d, 42), tables.fib_codebook(d, seed=42)
    x = _sin_vectors(16, d)
    st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert st == 0
    st, fast, _, _ = oracle_mod.fib_decode(payload, d, rot, cb)
    assert st == 0
    idx = np.zeros((16, 16), np.uint32)
    for v in range(16):
        rec = np.ascontiguousarray(payload[v, 2:])
        oracle_mod.lib().pkvo_unpack_bits(rec.ctypes.data_as(C.c_void_p), 16, 5,
                                          idx[v].ctypes.data_as(C.c_void_p))
    norms = payload[:, :2].copy().view(np.float16).astype(np.float64).ravel()
    rotated = cb.astype(np.float64)[idx].reshape(16, d)
    slow = (rotated @ rot) * norms[:, None]  # x = Pi^T y, fib-quant/src/rotation.rs:118-131
    assert np.max(np.abs(fast - slow)) <= 1e-4


def test_fib_single_and_batch_numerics_differ_only_in_normalisation(oracle_mod):
    # fib-quant/src/codec.rs:481 vs :607-609 -- n < 4 takes the single path under AUTO
    d = 64
    rot, cb = tables.haar_rotation(d, 42), tables.fib_codebook(d, seed=42)
    x = _sin_vectors(3, d)
    _, auto, _, _ = oracle_mod.fib_encode(x, rot, cb, numerics=0)
    _, single, _, _ = oracle_mod.fib_encode(x, rot, cb, numerics=2)
    assert np.array_equal(auto, single)
    x4 = _sin_vectors(4, d)
    _, auto4, _, _ = oracle_mod.fib_encode(x4, rot, cb, numerics=0)
    _, batch4, _, _ = oracle_mod.fib_encode(x4, rot, cb, numerics=1)
    assert np.array_equal(auto4, batch4)


def test_turbo_decode_is_deterministic_and_thread_invariant(oracle_mod):
    # turbo-quant/src/polar.rs:458-495 (batch == per-vector), tests/determinism.rs
    d = 64
    signs, qjl = tables.rademacher_signs(d, 1337), tables.qjl_matrix(d, 32, 1337)
    x = _sin_vectors(64, d)
    _, p1, _, _ = oracle_mod.turbo_encode(x, signs, qjl, nthreads=1)
    _, p4, _, _ = oracle_mod.turbo_encode(x, signs, qjl, nthreads=4)
    assert np.array_equal(p1, p4)
    _, a, _, _ = oracle_mod.turbo_decode(p1, d, signs, nthreads=1)
    one_by_one = np.concatenate([oracle_mod.turbo_decode(p1[i:i + 1], d, signs)[1] for i in range(64)])
    assert np.array_equal(a.view(np.uint32), one_by_one.view(np.uint32))
    other = tables.rademacher_signs(d, 1)
    assert not np.array_equal(signs, other)


def test_chacha_stream_of_the_reference_sign_generator():
    """turbo-quant/src/rotation.rs:152-155 draws its signs from ChaCha8Rng.  The block function is
    pinned by the published zero-key keystreams of ChaCha8 and ChaCha20 (same code, 8 / 20 rounds);
    the seeding and the bool rule are checked for their stated structure only."""
    import struct

    from provekv_b200 import tables

    ks8 = struct.pack("<16I", *tables.chacha_block([0] * 8, 0, 0, 8)).hex()
    ks20 = struct.pack("<16I", *tables.chacha_block([0] * 8, 0, 0, 20)).hex()
    assert ks8.startswith("3e00ef2f895f40d67f5bb8e81f09a5a12c840ec3ce9a7f3b181be188ef711a1e")
    assert ks20.startswith("76b8e0ada0f13d90405d6ae55386bd28bdd219b8a08ded1aa836efcc8b770dc7")
    # successive blocks only differ through the counter words
    assert tables.chacha_block([0] * 8, 1) != tables.chacha_block([0] * 8, 0)
    key = tables.seed_from_u64_key(42)
    assert len(key) == 8 and all(0 <= w < 1 << 32 for w in key) and key != tables.seed_from_u64_key(43)
    words = tables.chacha8_next_u32(42, 40)
    assert words[:16] == tables.chacha_block(key, 0) and words[16:32] == tables.chacha_block(key, 1)
    s = tables.reference_hadamard_signs(128, 42)
    assert s.dtype == np.float32 and set(np.unique(s)) == {-1.0, 1.0}
    expect = tables.chacha8_next_u32((42 + 0xA11CE55ED5A5EED5) & (2 ** 64 - 1), 128)
    assert [v > 0 for v in s] == [w >= 1 << 31 for w in expect]
    assert np.array_equal(s[:64], tables.reference_hadamard_signs(64, 42))  # a prefix of one stream


def test_hadamard_rotation_pins():
    """What gpu-backend/src/fallback.rs:312-364 states about hadamard_batch_cpu: a unit impulse comes out
    with magnitude 1/sqrt(dim) everywhere, a 768-vector is padded to 1024 and truncated back, equal inputs
    give equal outputs; and the LCG signs (:76-88) against a restatement in Python integers."""
    import oracle
    from provekv_b200 import tables
    d = np.zeros((2, 8), np.float32)
    d[:, 0] = 1.0
    out = oracle.hadamard_batch(d, 42)
    assert np.all(np.abs(np.abs(out) - 1.0 / np.sqrt(np.float32(8))) < 1e-5)
    z = np.zeros((1, 768), np.float32)
    z[0, 0] = 1.0
    out = oracle.hadamard_batch(z, 42)
    assert out.shape == (1, 768) and np.any(out != 0.0) and np.all(np.abs(out) == np.float32(1.0 / 32.0))
    v = np.arange(1.0, 9.0, dtype=np.float32)[None]
    assert np.array_equal(oracle.hadamard_batch(v, 42), oracle.hadamard_batch(v.copy(), 42))
    for seed in (0, 42, 2 ** 64 - 1, 0x9E3779B97F4A7C15):
        assert np.array_equal(oracle.hadamard_signs(128, seed), tables.lcg_hadamard_signs(128, seed))
    # the transform equals its matrix form, and that matrix is orthogonal
    m = tables.hadamard_rotation_matrix(128, 7)
    x = np.random.default_rng(0).standard_normal((5, 128)).astype(np.float32)
    assert np.abs(oracle.hadamard_batch(x, 7) - x.astype(np.float64) @ m.T).max() < 1e-6
    assert np.abs(m @ m.T - np.eye(128)).max() < 1e-7
    # the encoder built on it: the record of a vector is a function of that vector alone
    cb = tables.fib_codebook(64, seed=42)
    x = np.random.default_rng(1).standard_normal((40, 64)).astype(np.float32)
    st, a, _, _ = oracle.fib_encode_hadamard(x, 3, cb)
    st2, b, _, _ = oracle.fib_encode_hadamard(x[10:30], 3, cb, nthreads=3)
    assert st == 0 and st2 == 0 and np.array_equal(a[10:30], b)
