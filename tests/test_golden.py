"""Committed golden vectors (tests/golden/codec_golden.npz, made by make_golden.py):
the oracle must still reproduce them, and the CUDA path must reproduce them too."""
import os
import platform

import numpy as np
import pytest

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "codec_golden.npz"))
TURBO = [("qjl_f32", 1, 4, 0), ("qjl_log", 1, 4, 1), ("polar4_f32", 0, 4, 0)]


def _beq(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("d", [64, 128])
def test_oracle_reproduces_golden(oracle_mod, d):
    x, rot, cb = GOLD[f"x_{d}"], GOLD[f"rot_{d}"], GOLD[f"cb_{d}"]
    signs, qjl = GOLD[f"signs_{d}"], GOLD[f"qjl_{d}"]
    st, p, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert st == 0 and _beq(p, GOLD[f"fib_payload_{d}"])
    st, y, _, _ = oracle_mod.fib_decode(p, d, rot, cb)
    assert st == 0 and _beq(y, GOLD[f"fib_decoded_{d}"])
    same_libc = "-".join(platform.libc_ver()) == str(GOLD["libc"])
    for tag, mode, bits, rc in TURBO:
        for libm, lname in ((1, "portable"), (0, "platform")):
            if lname == "platform" and not same_libc:
                continue  # host-libm results are only pinned for the libc that produced them
            st, p, _, _ = oracle_mod.turbo_encode(x, signs, qjl if mode else None, bits=bits, mode=mode,
                                                  radii_codec=rc, libm_mode=libm)
            assert st == 0 and _beq(p, GOLD[f"turbo_{tag}_{lname}_payload_{d}"]), (tag, lname)
            st, y, _, _ = oracle_mod.turbo_decode(p, d, signs, bits=bits, mode=mode,
                                                  projections=32 if mode else 0, radii_codec=rc,
                                                  libm_mode=libm)
            assert st == 0 and _beq(y, GOLD[f"turbo_{tag}_{lname}_decoded_{d}"]), (tag, lname)


@pytest.mark.gpu
@pytest.mark.parametrize("d", [64, 128])
def test_cuda_reproduces_golden(d):
    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    x, rot, cb = GOLD[f"x_{d}"], GOLD[f"rot_{d}"], GOLD[f"cb_{d}"]
    signs, qjl = GOLD[f"signs_{d}"], GOLD[f"qjl_{d}"]
    fib = pk.FibProfile(d, rot, cb)
    wire = fib.encode_batch_compact(x)
    assert wire[19:] == GOLD[f"fib_payload_{d}"].tobytes()
    assert _beq(fib.decode_batch_compact(wire), GOLD[f"fib_decoded_{d}"])
    for tag, mode, bits, rc in TURBO:
        prof = pk.TurboProfile(d, bits, signs, qjl if mode else None, mode=mode, radii_codec=rc, seed=42)
        wire = prof.encode_batch_compact(x)
        assert wire[38:] == GOLD[f"turbo_{tag}_portable_payload_{d}"].tobytes(), tag
        assert _beq(prof.decode_batch_compact(wire), GOLD[f"turbo_{tag}_portable_decoded_{d}"]), tag
        if rc == L.RADII_F32 and _beq(GOLD[f"turbo_{tag}_portable_payload_{d}"],
                                      GOLD[f"turbo_{tag}_platform_payload_{d}"]):
            # the host libm put every pair of these vectors into the same bucket
            assert wire[38:] == GOLD[f"turbo_{tag}_platform_payload_{d}"].tobytes()


HGOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hadamard_golden.npz"))


def _wht_numpy(x, seed):
    """gpu-backend/src/fallback.rs:26-59 in NumPy binary32 arithmetic (power-of-two dim), written
    independently of the oracle's C: butterflies for step = 1, 2, 4, .., then the signs, then the scale."""
    from provekv_b200 import tables
    v = np.array(x, dtype=np.float32)
    d = v.shape[1]
    step = 1
    while step < d:
        w = v.reshape(-1, d // (2 * step), 2, step)
        a, b = w[:, :, 0, :].copy(), w[:, :, 1, :].copy()
        w[:, :, 0, :], w[:, :, 1, :] = a + b, a - b
        step *= 2
    v = v * tables.lcg_hadamard_signs(d, seed)
    return v * (np.float32(1.0) / np.sqrt(np.float32(d)))


@pytest.mark.parametrize("d", [64, 128])
def test_oracle_reproduces_hadamard_golden(oracle_mod, d):
    seed, x, cb = int(HGOLD["seed"]), HGOLD[f"x_{d}"], HGOLD[f"cb_{d}"]
    assert _beq(oracle_mod.hadamard_batch(x, seed), HGOLD[f"rotated_{d}"])
    assert _beq(_wht_numpy(x, seed), HGOLD[f"rotated_{d}"])
    for order in (0, 1):
        st, p, _, _ = oracle_mod.fib_encode_hadamard(x, seed, cb, argmin_order=order)
        assert st == 0 and _beq(p, HGOLD[f"fib_payload_{d}_order{order}"])


@pytest.mark.gpu
@pytest.mark.parametrize("d", [64, 128])
def test_cuda_reproduces_hadamard_golden(d):
    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    seed, x, cb = int(HGOLD["seed"]), HGOLD[f"x_{d}"], HGOLD[f"cb_{d}"]
    for order in (0, 1):
        prof = pk.FibProfile(d, None, cb, argmin_order=order, hadamard_seed=seed)   # AUTO numerics: >= 16 vectors
        assert prof.encode_batch_compact(x)[19:] == HGOLD[f"fib_payload_{d}_order{order}"].tobytes()
