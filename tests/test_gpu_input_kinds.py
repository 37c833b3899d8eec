"""Byte and word parity with the oracle over kinds of input the seeded KV generator does not produce:
per-channel scales, outlier channels, global scales from 1e-6 to 1e3, fp16-valued inputs and a coarse
grid (many equal coordinates and exact zeros, hence exact ties in the angle and codeword decisions)."""
import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import tables

pytestmark = pytest.mark.gpu

KINDS = ["channel_scale", "outlier_channels", "global_scale", "fp16_valued", "coarse_grid"]


def _inputs(kind, n, dim, seed):
    rng = np.random.default_rng(1000 * dim + seed)
    x = rng.standard_normal((n, dim)).astype(np.float32)
    if kind == "channel_scale":
        x *= np.exp(0.5 * rng.standard_normal((1, dim))).astype(np.float32)
    elif kind == "outlier_channels":
        x[:, rng.integers(0, dim, 2)] *= 20.0
    elif kind == "global_scale":
        x *= np.float32(10.0 ** rng.uniform(-6, 3))
    elif kind == "fp16_valued":
        x = x.astype(np.float16).astype(np.float32)
    elif kind == "coarse_grid":
        x = np.round(x * 4) / 4
    x = np.ascontiguousarray(x, np.float32)
    x[~np.any(x != 0, axis=1)] = 1.0  # the fib encoder refuses all-zero vectors
    return x


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("kind", KINDS)
def test_every_codec_on_every_kind_of_input(oracle_mod, dim, kind):
    n = 60_000 if dim == 64 else 30_000
    rot, cb = tables.haar_rotation(dim, 42), tables.fib_codebook(dim, seed=42)
    signs, qjl = tables.rademacher_signs(dim, 42), tables.qjl_matrix(dim, 32, 42)
    profiles = {"fib": pk.FibProfile(dim, rot, cb), "turbo": pk.TurboProfile(dim, 4, signs, qjl, seed=42),
                "turbo_lossy": pk.TurboProfile(dim, 4, signs, qjl, seed=42, radii_codec=L.RADII_BLOCK_LOG_U8)}
    for seed in (0, 1):
        x = _inputs(kind, n, dim, seed)
        for name, prof in profiles.items():
            got = prof.encode_batch_compact(x)
            if name == "fib":
                st, pay, _, _ = oracle_mod.fib_encode(x, rot, cb, nthreads=8)
                hdr = L.FB2_HEADER_BYTES
            else:
                st, pay, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=4, mode=1, radii_codec=prof.radii_codec,
                                                        libm_mode=oracle_mod.LIBM_PORTABLE, nthreads=8)
                hdr = L.TQB1_HEADER_BYTES
            assert st == 0
            have, want = np.frombuffer(got, np.uint8)[hdr:].reshape(n, -1), pay.reshape(n, -1)
            assert np.array_equal(have, want), \
                f"{name} {kind} seed {seed}: {(have != want).any(axis=1).sum()} records differ"
            dec = prof.decode_batch_compact(got)
            if name == "fib":
                st, ref, _, _ = oracle_mod.fib_decode(pay, dim, rot, cb, nthreads=8)
            else:
                st, ref, _, _ = oracle_mod.turbo_decode(pay, dim, signs, bits=4, mode=1, projections=32,
                                                        radii_codec=prof.radii_codec,
                                                        libm_mode=oracle_mod.LIBM_PORTABLE, nthreads=8)
            assert st == 0 and np.array_equal(dec.view(np.uint32).reshape(-1), ref.view(np.uint32).reshape(-1))
