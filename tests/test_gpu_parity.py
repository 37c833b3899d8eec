"""CUDA kernels vs the CPU oracle on the same seeded inputs, through the C ABI.

Bar: wire bytes bit-exact; decoded f32 bit-exact against the oracle's portable
libm mode and within 1e-6 relative / 1e-7 absolute of its platform libm mode
(the tolerance BASELINE.json states for decoded values).
"""
import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import tables

from kvgen import synthetic_kv

pytestmark = pytest.mark.gpu

SEED = 42


@pytest.fixture(scope="module")
def fib_tables():
    out = {}
    for d in (64, 128):
        out[d] = (tables.haar_rotation(d, SEED), tables.fib_codebook(d, seed=SEED))
    return out


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("n", [1, 3, 4, 63, 64, 129, 1000, 4099])
def test_fib_encode_bytes_match_oracle(oracle_mod, fib_tables, dim, n):
    rot, cb = fib_tables[dim]
    x = synthetic_kv(n, dim, seed=n)
    prof = pk.FibProfile(dim, rot, cb)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert st == 0
    want = oracle_mod.fb2_header(dim, n) + payload.tobytes()
    assert len(got) == 19 + n * prof.record_bytes
    assert got == want


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("n", [1, 5, 127, 128, 129, 2000])
def test_fib_decode_matches_oracle_bitwise(oracle_mod, fib_tables, dim, n):
    rot, cb = fib_tables[dim]
    x = synthetic_kv(n, dim, seed=100 + n)
    st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb)
    wire = oracle_mod.fb2_header(dim, n) + payload.tobytes()
    prof = pk.FibProfile(dim, rot, cb)
    got = prof.decode_batch_compact(wire)
    st, want, _, _ = oracle_mod.fib_decode(payload, dim, rot, cb)
    assert st == 0
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("order", [L.ARGMIN_PAIRWISE, L.ARGMIN_SEQUENTIAL])
@pytest.mark.parametrize("norm_format", [L.NORM_FP16, L.NORM_F32])
@pytest.mark.parametrize("ncw", [32, 31, 17])
def test_fib_variants(oracle_mod, fib_tables, order, norm_format, ncw):
    dim, n = 64, 777
    rot, cb = fib_tables[dim]
    cb = cb[:ncw]
    x = synthetic_kv(n, dim, seed=7)
    prof = pk.FibProfile(dim, rot, cb, norm_format=norm_format, argmin_order=order)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb, norm_format=norm_format, argmin_order=order)
    assert st == 0
    assert got == oracle_mod.fb2_header(dim, n, n_codewords=ncw, norm_format=norm_format) + payload.tobytes()
    dec = prof.decode_batch_compact(got)
    st, want, _, _ = oracle_mod.fib_decode(payload, dim, rot, cb, norm_format=norm_format)
    assert np.array_equal(dec.view(np.uint32), want.view(np.uint32))


TURBO_CASES = [
    # (bits, mode, projections, radii_codec)
    (4, L.TURBO_POLAR_WITH_QJL, 32, L.RADII_F32),          # proveKV "turbo b=4": polar 3 bit + 32 QJL
    (4, L.TURBO_POLAR_WITH_QJL, 32, L.RADII_BLOCK_LOG_U8),
    (4, L.TURBO_POLAR_ONLY, 0, L.RADII_F32),               # literal 4-bit angles
    (4, L.TURBO_POLAR_ONLY, 0, L.RADII_BLOCK_LOG_U8),
    (8, L.TURBO_POLAR_WITH_QJL, 32, L.RADII_F32),          # legacy turbo_8bit
    (2, L.TURBO_POLAR_WITH_QJL, 64, L.RADII_BLOCK_LOG_U8),
]


def _turbo_tables(dim, m):
    return tables.rademacher_signs(dim, SEED), (tables.qjl_matrix(dim, m, SEED) if m else None)


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("case", TURBO_CASES)
@pytest.mark.parametrize("n", [1, 127, 128, 129, 1500])
def test_turbo_encode_bytes_match_oracle(oracle_mod, dim, case, n):
    bits, mode, m, rc = case
    signs, qjl = _turbo_tables(dim, m)
    x = synthetic_kv(n, dim, seed=n + bits)
    prof = pk.TurboProfile(dim, bits, signs, qjl, mode=mode, radii_codec=rc, seed=SEED)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=bits, mode=mode, radii_codec=rc,
                                               libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    want = oracle_mod.tqb1_header(dim, bits, mode, m, rc, SEED, n) + payload.tobytes()
    assert len(got) == len(want)
    assert got == want


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("case", TURBO_CASES)
@pytest.mark.parametrize("n", [1, 129, 1500])
def test_turbo_decode_matches_oracle(oracle_mod, dim, case, n):
    bits, mode, m, rc = case
    signs, qjl = _turbo_tables(dim, m)
    x = synthetic_kv(n, dim, seed=3 * n + bits)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=bits, mode=mode, radii_codec=rc)
    wire = oracle_mod.tqb1_header(dim, bits, mode, m, rc, SEED, n) + payload.tobytes()
    prof = pk.TurboProfile(dim, bits, signs, qjl, mode=mode, radii_codec=rc, seed=SEED)
    got = prof.decode_batch_compact(wire)
    st, want, _, _ = oracle_mod.turbo_decode(payload, dim, signs, bits=bits, mode=mode, projections=m,
                                            radii_codec=rc, libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # Against the host libm (what the Rust reference calls on this machine).  Without the
    # BlockLogU8 radii no libm call is left on the decode path (the cos/sin table is an
    # input), so the result is bit-identical.  With them, expf differs by <= 1 ulp per
    # radius between libms; after the 64-term butterflies a few 1e-5 of the elements
    # (those that cancel to near zero) fall outside the literal 1e-6 rel / 1e-7 abs, so the
    # bound is taken relative to the largest element of the vector.
    st, plat, _, _ = oracle_mod.turbo_decode(payload, dim, signs, bits=bits, mode=mode, projections=m,
                                            radii_codec=rc, libm_mode=oracle_mod.LIBM_PLATFORM)
    if rc == L.RADII_F32:
        assert np.array_equal(got.view(np.uint32), plat.view(np.uint32))
    else:
        err = np.abs(got - plat)
        assert np.all(err.max(axis=1) <= 1e-6 * np.abs(plat).max(axis=1))
        assert np.mean(err > 1e-7 + 1e-6 * np.abs(plat)) < 1e-3


def test_turbo_sign_tiers_with_degenerate_projection_rows(oracle_mod):
    """QJL matrix with all-zero rows, rows of magnitude 1e-30 and rows that are exact copies or
    negatives of others: every dot with a zero row is exactly 0 (sign bit 1), tiny rows give dots far
    below any bound relative to nothing -- all of them miss the tensor-core and binary32 tiers and
    are settled by the exact sequence, for every vector, so the per-warp list overflows as well."""
    dim, n, m = 64, 3000, 32
    signs, qjl = _turbo_tables(dim, m)
    q = np.array(qjl, dtype=np.float32).reshape(m, dim).copy()
    q[0:6] = 0.0
    q[6:12] *= np.float32(1e-30)
    q[12] = q[13]
    q[14] = -q[15]
    x = synthetic_kv(n, dim, seed=91)
    x[5] = 0.0                      # an all-zero vector: zero residual, every sign bit 1
    x[6] = x[7]
    prof = pk.TurboProfile(dim, 4, signs, q, mode=L.TURBO_POLAR_WITH_QJL, seed=SEED)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, q, bits=4, mode=L.TURBO_POLAR_WITH_QJL,
                                               radii_codec=L.RADII_F32, libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    want = payload.reshape(n, -1)
    have = np.frombuffer(got, np.uint8)[L.TQB1_HEADER_BYTES:].reshape(n, -1)
    assert np.array_equal(have, want)
    assert np.all(have[5, -4:] == 0xff) and np.all(have[:, -4] & 0x3f == 0x3f)  # zero rows -> bit 1


def test_fib_blocks_placed_between_codewords(oracle_mod, fib_tables):
    """Vectors whose normalised, rotated 4-blocks sit on (and within 1e-7 .. 1e-3 of) the bisector
    between two codewords: where those two are the nearest, the top-2 gap is at or below every
    tier's bound, so the decision falls through the tensor-core tier and the binary32 tier to the
    exact f64 kernel -- whose answer must be the oracle's, including the lowest-index rule."""
    dim, n, B = 64, 4096, 16
    rot, cb = fib_tables[dim]
    c = np.asarray(cb, np.float64)
    rng = np.random.default_rng(17)
    i = rng.integers(0, 32, size=(n, B))
    j = (i + rng.integers(1, 32, size=(n, B))) % 32
    ci, cj = c[i], c[j]                                   # [n, B, 4]
    dn = ((ci - cj) ** 2).sum(-1)
    t = np.full((n, B), 0.5)
    for _ in range(40):   # the blocks of y / |y| on the bisectors: fixed point in the scale 1 / |y|
        y = t[..., None] * ci + (1.0 - t[..., None]) * cj
        s = 1.0 / np.sqrt((y ** 2).sum((1, 2)))[:, None]
        t = (((ci ** 2).sum(-1) - (cj ** 2).sum(-1)) / (2.0 * s) - (cj * (ci - cj)).sum(-1)) / dn
    t += rng.choice([0.0, 1e-7, -1e-7, 1e-5, -1e-5, 1e-3, -1e-3], size=(n, B))
    y = (t[..., None] * ci + (1.0 - t[..., None]) * cj).reshape(n, dim)
    x = (y @ np.asarray(rot, np.float64)).astype(np.float32) * np.float32(3.0)   # x = M^T y, any norm
    prof = pk.FibProfile(dim, rot, cb)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert st == 0
    assert got[L.FB2_HEADER_BYTES:] == payload.tobytes()


@pytest.mark.parametrize("bits,mode", [(4, L.TURBO_POLAR_WITH_QJL), (4, L.TURBO_POLAR_ONLY), (8, L.TURBO_POLAR_WITH_QJL)])
def test_turbo_pairs_exactly_on_sector_boundaries(oracle_mod, bits, mode):
    """Rotated pairs placed exactly on the bucket boundaries (axes, diagonals, zero pairs): with
    small-integer rotated coordinates the inverse transform is exact in binary32, so the encoder's
    forward transform lands on the integers again and every such pair is a knife-edge for
    floor((atan2f(b, a) + pi) / (2 pi) * L): the shortcut must hand all of them to the exact path."""
    dim, n = 64, 2048
    m = 32 if mode == L.TURBO_POLAR_WITH_QJL else 0
    signs, qjl = _turbo_tables(dim, m)
    rng = np.random.default_rng(5)
    k = rng.integers(1, 5, size=(n, dim // 2)).astype(np.float64)
    kind = rng.integers(0, 10, size=(n, dim // 2))
    a = np.select([kind == 0, kind == 1, kind == 2, kind == 3, kind == 4, kind == 5, kind == 6, kind == 7, kind == 8],
                  [k, 0 * k, -k, 0 * k, k, -k, -k, k, 0 * k], default=rng.integers(-4, 5, size=k.shape))
    b = np.select([kind == 0, kind == 1, kind == 2, kind == 3, kind == 4, kind == 5, kind == 6, kind == 7, kind == 8],
                  [0 * k, k, 0 * k, -k, k, k, -k, -k, 0 * k], default=rng.integers(-4, 5, size=k.shape))
    y = np.stack([a, b], axis=-1).reshape(n, dim)
    h = np.array([[1.0]])
    while h.shape[0] < dim:
        h = np.block([[h, h], [h, -h]])
    x = ((y @ h) / 8.0 * np.asarray(signs, np.float64)[None, :]).astype(np.float32)  # exact: x = D H y / sqrt(d)
    prof = pk.TurboProfile(dim, bits, signs, qjl, mode=mode, seed=SEED)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=bits, mode=mode, radii_codec=L.RADII_F32,
                                               libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    assert got[L.TQB1_HEADER_BYTES:] == payload.tobytes()
    # the construction really is exact: the radii on the wire are the integer hypotenuses
    rec = np.frombuffer(got, np.uint8)[L.TQB1_HEADER_BYTES:].reshape(n, -1)
    radii = rec[:, :dim * 2].copy().view(np.float32)
    assert np.array_equal(radii, np.sqrt(a * a + b * b).astype(np.float32))


@pytest.mark.parametrize("dim", [64, 128])
def test_polar_only_profile_on_the_reference_sign_stream(oracle_mod, dim):
    """A polar-only quantizer needs nothing from the seed but the Hadamard signs; with
    sign_stream="chacha8" they come from the reference's own generator stream."""
    n = 700
    prof = pk.TurboProfile.from_seed(dim, 4, 0, SEED, mode=L.TURBO_POLAR_ONLY, sign_stream="chacha8")
    signs = tables.reference_hadamard_signs(dim, SEED)
    assert np.array_equal(prof.signs, signs) and not np.array_equal(signs, tables.rademacher_signs(dim, SEED))
    x = synthetic_kv(n, dim, seed=dim)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, None, bits=4, mode=L.TURBO_POLAR_ONLY,
                                               radii_codec=L.RADII_F32, libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    assert got == oracle_mod.tqb1_header(dim, 4, L.TURBO_POLAR_ONLY, 0, L.RADII_F32, SEED, n) + payload.tobytes()
    st, want, _, _ = oracle_mod.turbo_decode(payload, dim, signs, bits=4, mode=L.TURBO_POLAR_ONLY, projections=0,
                                            radii_codec=L.RADII_F32, libm_mode=oracle_mod.LIBM_PORTABLE)
    assert np.array_equal(prof.decode_batch_compact(got).view(np.uint32), want.view(np.uint32))


def _c2_vectors():
    return synthetic_kv(344_064, 64, seed=2, groups=1536)


@pytest.mark.parametrize("lossy", [False, True])
def test_c2_bytes_against_the_host_libm_oracle(oracle_mod, lossy):
    """What the Rust reference would write on this machine (oracle in PLATFORM mode: host atan2f, logf,
    expf) against the GPU, C2 at full size.
    BlockLogU8 radii: a profile created with LIBM_PLATFORM reproduces the host's logf bit for bit, so the
    radius bytes (codes, min, max) of every vector are equal; a LIBM_PORTABLE profile differs in a few
    bytes per thousand vectors (the one-unit deviations of glibc's logf), counted and bounded here.
    Angle buckets: the kernels take atan2f correctly rounded, glibc's differs by a unit on 16 % of the
    arguments, which moves a bucket only when the angle sits within that unit of a bucket boundary:
    about 1e-7 of the pairs, i.e. a handful of the 344,064 vectors (their QJL signs follow)."""
    dim, m = 64, 32
    rc = L.RADII_BLOCK_LOG_U8 if lossy else L.RADII_F32
    signs, qjl = _turbo_tables(dim, m)
    x = _c2_vectors()
    n = x.shape[0]
    st, plat, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=4, mode=1, radii_codec=rc,
                                            libm_mode=oracle_mod.LIBM_PLATFORM, nthreads=8)
    assert st == 0
    plat = plat.reshape(n, -1)
    radii_bytes = 32 + 8 if lossy else 128
    for libm in ((L.LIBM_PLATFORM, L.LIBM_PORTABLE) if lossy else (L.LIBM_PORTABLE,)):
        prof = pk.TurboProfile(dim, 4, signs, qjl, radii_codec=rc, seed=SEED, libm=libm)
        got = np.frombuffer(prof.encode_batch_compact(x), np.uint8)[L.TQB1_HEADER_BYTES:].reshape(n, -1)
        radii_diff = (got[:, :radii_bytes] != plat[:, :radii_bytes])
        angle_diff = (got[:, radii_bytes:radii_bytes + 12] != plat[:, radii_bytes:radii_bytes + 12]).any(axis=1)
        print(f"lossy={lossy} libm={libm}: {int(radii_diff.sum())} radius bytes in {int(radii_diff.any(axis=1).sum())} "
              f"vectors, {int(angle_diff.sum())} vectors with another angle bucket, of {n}")
        assert angle_diff.sum() <= 8
        if not lossy or libm == L.LIBM_PLATFORM:
            assert radii_diff.sum() == 0
            assert (got != plat).any(axis=1).sum() == angle_diff.sum()  # nothing else differs
        else:
            assert 0 < radii_diff.sum() <= 0.02 * n  # ~5 bytes per 1000 vectors
        if lossy and libm == L.LIBM_PLATFORM:
            # decode with the host's expf: bit-identical to the oracle's platform decode
            wire = oracle_mod.tqb1_header(dim, 4, 1, m, rc, SEED, n) + plat.tobytes()
            dec = prof.decode_batch_compact(wire)
            st, want, _, _ = oracle_mod.turbo_decode(plat, dim, signs, bits=4, mode=1, projections=m, radii_codec=rc,
                                                    libm_mode=oracle_mod.LIBM_PLATFORM, nthreads=8)
            assert st == 0 and np.array_equal(dec.view(np.uint32), want.view(np.uint32))
