"""Regenerates tests/golden/codec_golden.npz and tests/golden/hadamard_golden.npz.

The reference is Rust and cannot run here, so these vectors are outputs of the
CPU oracle (oracle/pkv_oracle.c), frozen so that (a) a later change of the oracle
or of the portable math shows up as a diff against committed bytes and (b) the
CUDA path can be checked on a machine where only the fixtures travel.  Inputs are
the closed-form vectors the reference's own tests use
(sin((i*d + j) * 0.013), fib-quant/src/codec.rs:1099-1105) plus seeded synthetic
KV rows; tables come from provekv_b200.tables.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from kvgen import synthetic_kv  # noqa: E402
from provekv_b200 import tables  # noqa: E402

SEED = 42


def inputs(n, d):
    i = np.arange(n // 2)[:, None]
    j = np.arange(d)[None, :]
    a = np.sin((i * d + j) * 0.013).astype(np.float32)
    return np.concatenate([a, synthetic_kv(n - n // 2, d, seed=d)])


def main():
    out = {}
    for d, n in ((64, 24), (128, 12)):
        x = inputs(n, d)
        rot, cb = tables.haar_rotation(d, SEED), tables.fib_codebook(d, seed=SEED)
        signs, qjl = tables.rademacher_signs(d, SEED), tables.qjl_matrix(d, 32, SEED)
        out[f"x_{d}"], out[f"rot_{d}"], out[f"cb_{d}"] = x, rot, cb
        out[f"signs_{d}"], out[f"qjl_{d}"] = signs, qjl
        st, p, _, _ = oracle.fib_encode(x, rot, cb)
        assert st == 0
        out[f"fib_payload_{d}"] = p
        st, y, _, _ = oracle.fib_decode(p, d, rot, cb)
        assert st == 0
        out[f"fib_decoded_{d}"] = y
        for tag, mode, bits, rc in (("qjl_f32", 1, 4, 0), ("qjl_log", 1, 4, 1), ("polar4_f32", 0, 4, 0)):
            for libm, lname in ((oracle.LIBM_PORTABLE, "portable"), (oracle.LIBM_PLATFORM, "platform")):
                st, p, _, _ = oracle.turbo_encode(x, signs, qjl if mode else None, bits=bits, mode=mode,
                                                  radii_codec=rc, libm_mode=libm)
                assert st == 0
                out[f"turbo_{tag}_{lname}_payload_{d}"] = p
                st, y, _, _ = oracle.turbo_decode(p, d, signs, bits=bits, mode=mode,
                                                  projections=32 if mode else 0, radii_codec=rc,
                                                  libm_mode=libm)
                assert st == 0
                out[f"turbo_{tag}_{lname}_decoded_{d}"] = y
    import platform
    out["libc"] = np.array("-".join(platform.libc_ver()))
    np.savez_compressed(os.path.join(HERE, "codec_golden.npz"), **out)
    print("wrote", len(out), "arrays")
    hadamard()


HADAMARD_SEED = 0x9E3779B97F4A7C15


def hadamard():
    """hadamard_golden.npz: the Walsh-Hadamard rotation of the reference's `gpu` build (gpu-backend/src/
    fallback.rs:12-88) on the same inputs, and the fib records encoded through it (fib-quant/src/codec.rs:612-656)."""
    out = {"seed": np.array(HADAMARD_SEED, dtype=np.uint64)}
    for d, n in ((64, 24), (128, 20)):
        x = inputs(n, d)
        cb = tables.fib_codebook(d, seed=SEED)
        out[f"x_{d}"], out[f"cb_{d}"] = x, cb
        out[f"rotated_{d}"] = oracle.hadamard_batch(x, HADAMARD_SEED)
        for order in (0, 1):
            st, p, _, _ = oracle.fib_encode_hadamard(x, HADAMARD_SEED, cb, argmin_order=order)
            assert st == 0
            out[f"fib_payload_{d}_order{order}"] = p
    np.savez_compressed(os.path.join(HERE, "hadamard_golden.npz"), **out)
    print("wrote", len(out), "arrays (hadamard)")


if __name__ == "__main__":
    main()
