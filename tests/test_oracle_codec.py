"""Oracle behaviour: round trips, error semantics and edge cases of the reference
(empty and ragged batches, non-finite input, zero vectors, out-of-range norms,
corrupted payloads)."""
import numpy as np
import pytest

from provekv_b200 import _lib as L
from provekv_b200 import tables

from kvgen import synthetic_kv


@pytest.fixture(scope="module")
def fib64():
    return tables.haar_rotation(64, 42), tables.fib_codebook(64, seed=42)


@pytest.fixture(scope="module")
def turbo64():
    return tables.rademacher_signs(64, 42), tables.qjl_matrix(64, 32, 42)


def test_fib_roundtrip_quality(oracle_mod, fib64):
    rot, cb = fib64
    x = synthetic_kv(4000, 64, seed=1)
    st, p, _, _ = oracle_mod.fib_encode(x, rot, cb, nthreads=4)
    assert st == 0
    st, y, _, _ = oracle_mod.fib_decode(p, 64, rot, cb, nthreads=4)
    assert st == 0
    rel = np.sum((x - y) ** 2) / np.sum(x ** 2)
    assert 0.05 < rel < 0.4  # 1.25 bits per coordinate: lossy but informative
    cos = np.sum(x * y, 1) / (np.linalg.norm(x, axis=1) * np.linalg.norm(y, axis=1))
    assert cos.mean() > 0.8


@pytest.mark.parametrize("mode,bits,rc", [(1, 4, 0), (1, 4, 1), (0, 4, 0), (0, 4, 1), (1, 8, 0)])
def test_turbo_roundtrip_quality(oracle_mod, turbo64, mode, bits, rc):
    signs, qjl = turbo64
    x = synthetic_kv(2000, 64, seed=2)
    st, p, _, _ = oracle_mod.turbo_encode(x, signs, qjl if mode else None, bits=bits, mode=mode,
                                          radii_codec=rc)
    assert st == 0
    st, y, _, _ = oracle_mod.turbo_decode(p, 64, signs, bits=bits, mode=mode,
                                          projections=32 if mode else 0, radii_codec=rc)
    assert st == 0
    rel = np.sum((x - y) ** 2) / np.sum(x ** 2)
    pb = bits - 1 if mode else bits
    assert rel < {3: 0.25, 4: 0.07, 7: 0.002}[pb]


def test_fib_empty_batch_is_an_error(oracle_mod, fib64):
    rot, cb = fib64
    st, _, _, _ = oracle_mod.fib_encode(np.zeros((0, 64), np.float32), rot, cb)
    assert st == L.ERR_EMPTY_BATCH  # fib-quant/src/codec.rs:226


def test_fib_first_error_wins(oracle_mod, fib64):
    rot, cb = fib64
    x = synthetic_kv(100, 64, seed=3)
    x[70, 5] = np.nan
    x[40] = 0.0
    x[90, 0] = np.inf
    st, _, code, idx = oracle_mod.fib_encode(x, rot, cb, nthreads=3)
    assert (st, code, idx) == (L.VEC_ZERO_NORM, L.VEC_ZERO_NORM, 40)
    x[40, 0] = 1.0
    st, _, code, idx = oracle_mod.fib_encode(x, rot, cb)
    assert (code, idx) == (L.VEC_NONFINITE_INPUT, 70)


def test_fib_norm_range_is_a_second_pass_error(oracle_mod, fib64):
    rot, cb = fib64
    x = synthetic_kv(50, 64, seed=4)
    x[10] *= 1e5      # norm > 65504: not representable in fp16 (codec.rs:1003)
    x[30, 0] = np.nan  # first-pass error at a later index still wins (codec.rs:594-610 run first)
    st, _, code, idx = oracle_mod.fib_encode(x, rot, cb)
    assert (code, idx) == (L.VEC_NONFINITE_INPUT, 30)
    x[30, 0] = 1.0
    st, _, code, idx = oracle_mod.fib_encode(x, rot, cb)
    assert (code, idx) == (L.VEC_NORM_RANGE, 10)
    x[10] *= 1e-15    # underflows to fp16 zero
    st, _, code, idx = oracle_mod.fib_encode(x, rot, cb)
    assert (code, idx) == (L.VEC_NORM_RANGE, 10)
    st, _, code, idx = oracle_mod.fib_encode(x, rot, cb, norm_format=L.NORM_F32)
    assert st == 0


def test_fib_decode_rejections(oracle_mod, fib64):
    rot, cb = fib64
    x = synthetic_kv(20, 64, seed=5)
    st, p, _, _ = oracle_mod.fib_encode(x, rot, cb[:20])  # N = 20 -> indices 20..31 invalid
    assert st == 0
    bad = p.copy()
    bad[7, 2] |= 0x1f  # first index = 31
    st, _, code, idx = oracle_mod.fib_decode(bad, 64, rot, cb[:20])
    assert (code, idx) == (L.VEC_INDEX_RANGE, 7)
    bad = p.copy()
    bad[3, 0:2] = 0  # fp16 zero norm
    bad[9, 0:2] = [0x00, 0x7c]  # fp16 +inf
    st, _, code, idx = oracle_mod.fib_decode(bad, 64, rot, cb[:20])
    assert (code, idx) == (L.VEC_BAD_NORM, 3)
    bad = p.copy()
    bad[5, 1] |= 0x80  # negative norm
    st, _, code, idx = oracle_mod.fib_decode(bad, 64, rot, cb[:20])
    assert (code, idx) == (L.VEC_BAD_NORM, 5)


def test_fib_padding_bits_rejected_small_dim(oracle_mod):
    d = 8  # 2 blocks x 5 bits = 10 bits -> 6 padding bits in the second byte
    rot, cb = tables.haar_rotation(d, 1), tables.fib_codebook(d, seed=1, training_samples=256)
    x = synthetic_kv(6, d, seed=6)
    st, p, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert st == 0 and p.shape == (6, 4)
    assert oracle_mod.fib_decode(p, d, rot, cb)[0] == 0
    bad = p.copy()
    bad[2, 3] |= 0x40
    st, _, code, idx = oracle_mod.fib_decode(bad, d, rot, cb)
    assert (code, idx) == (L.VEC_PADDING_BITS, 2)


def test_turbo_zero_vector_is_allowed(oracle_mod, turbo64):
    # turbo-quant/src/polar.rs:526-533: zero input encodes (radii 0)
    signs, qjl = turbo64
    x = np.zeros((5, 64), np.float32)
    for rc in (0, 1):
        st, p, _, _ = oracle_mod.turbo_encode(x, signs, qjl, radii_codec=rc)
        assert st == 0
        st, y, _, _ = oracle_mod.turbo_decode(p, 64, signs, radii_codec=rc)
        assert st == 0
        assert np.all(np.abs(y) < 1e-30)


def test_turbo_errors(oracle_mod, turbo64):
    signs, qjl = turbo64
    x = synthetic_kv(30, 64, seed=7)
    x[12, 63] = -np.inf
    st, _, code, idx = oracle_mod.turbo_encode(x, signs, qjl)
    assert (code, idx) == (L.VEC_NONFINITE_INPUT, 12)
    x[12, 63] = 3e38  # finite input, the butterflies overflow -> non-finite radius (polar.rs:127)
    x[12, 62] = 3e38
    st, _, code, idx = oracle_mod.turbo_encode(x, signs, qjl)
    assert (code, idx) == (L.VEC_BAD_RADIUS, 12)
    assert oracle_mod.turbo_encode(np.zeros((0, 64), np.float32), signs, qjl)[0] == L.ERR_EMPTY_BATCH
    x = synthetic_kv(30, 64, seed=8)
    st, p, _, _ = oracle_mod.turbo_encode(x, signs, qjl)
    bad = p.copy()
    bad[4, 3] = 0xff  # radius 0 becomes negative / NaN pattern
    bad[4, 2] = 0xff
    st, _, code, idx = oracle_mod.turbo_decode(bad, 64, signs)
    assert (code, idx) == (L.VEC_BAD_RADIUS, 4)
    st, p, _, _ = oracle_mod.turbo_encode(x, signs, qjl, radii_codec=1)
    bad = p.copy()
    bad[6, 32:36], bad[6, 36:40] = p[6, 36:40], p[6, 32:36]  # min > max (radius.rs:170-177)
    st, _, code, idx = oracle_mod.turbo_decode(bad, 64, signs, radii_codec=1)
    assert (code, idx) == (L.VEC_BAD_RADIUS_RANGE, 6)
    bad = p.copy()
    bad[8, 36:40] = np.frombuffer(np.float32(200.0).tobytes(), np.uint8)  # exp overflows -> inf radius
    bad[8, 0] = 255
    st, _, code, idx = oracle_mod.turbo_decode(bad, 64, signs, radii_codec=1)
    assert (code, idx) == (L.VEC_BAD_RADIUS, 8)


def test_lossy_radii_within_five_percent(oracle_mod, turbo64):
    # turbo-quant/src/wire.rs:940-944: BlockLogU8 radii within 5 %, angles and signs exact
    signs, qjl = turbo64
    x = synthetic_kv(500, 64, seed=9)
    _, exact, _, _ = oracle_mod.turbo_encode(x, signs, qjl, radii_codec=0)
    _, lossy, _, _ = oracle_mod.turbo_encode(x, signs, qjl, radii_codec=1)
    assert np.array_equal(exact[:, 128:], lossy[:, 40:])  # angle + sign bytes identical
    r = exact[:, :128].copy().view(np.float32)
    q = lossy[:, :32].astype(np.float32)
    mn = lossy[:, 32:36].copy().view(np.float32)
    mx = lossy[:, 36:40].copy().view(np.float32)
    back = np.exp(mn + (mx - mn) * (q / 255.0))
    assert np.max(np.abs(back - r) / np.maximum(r, 1e-6)) < 0.05


def test_oracle_scoring_against_reconstruction_and_host_mirror(oracle_mod):
    """Compressed-domain scores (turbo.rs:340-381): the polar part equals the inner product with the
    reconstruction (the rotation is orthonormal), the QJL part adds sqrt(pi/2)/m * sum of +-p_j, and
    the package's host-side prepare_query reproduces the oracle's rotated / projected query bits."""
    import provekv_b200 as pk
    from provekv_b200 import tables

    d, n = 64, 500
    signs, qjl = tables.rademacher_signs(d, 42), tables.qjl_matrix(d, 32, 42)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n, d)).astype(np.float32)
    q = rng.standard_normal(d).astype(np.float32)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=4, mode=1, radii_codec=0)
    assert st == 0
    st, rotated, projected = oracle_mod.turbo_prepare_query(q, signs, qjl)
    assert st == 0

    class _Stub:  # prepare_query only reads these fields; no GPU library needed
        dim, signs, qjl = d, None, None
    stub = _Stub()
    stub.signs, stub.qjl = signs, qjl
    r2, p2 = pk.TurboProfile.prepare_query(stub, q)
    assert np.array_equal(r2.view(np.uint32), rotated.view(np.uint32))
    assert np.array_equal(p2.view(np.uint32), projected.view(np.uint32))

    st, full, _, _ = oracle_mod.turbo_score(payload, d, rotated, projected)
    st, polar, _, _ = oracle_mod.turbo_score(payload, d, rotated, np.zeros(32, np.float32))
    st, dec, _, _ = oracle_mod.turbo_decode(payload, d, signs)
    assert np.allclose(polar, dec @ q, rtol=1e-5, atol=1e-4)
    sign_bits = np.unpackbits(payload.reshape(n, -1)[:, -4:], axis=1, bitorder="little").astype(np.float32) * 2 - 1
    corr = np.float32(np.sqrt(np.float32(np.pi) / np.float32(2))) / np.float32(32) * (sign_bits @ projected)
    assert np.allclose(full - polar, corr, rtol=1e-4, atol=1e-4)
