"""The Hadamard-rotation fib encoder (what the reference's `gpu` build emits from encode_batch,
fib-quant/src/codec.rs:612-656 with gpu-backend/src/fallback.rs:12-88) against the oracle, byte for byte."""
import numpy as np
import pytest

from provekv_b200 import _lib as L
from provekv_b200 import tables
from provekv_b200.profiles import FibProfile, encode_batches_compact
from kvgen import synthetic_kv

pytestmark = pytest.mark.gpu
H = L.FB2_HEADER_BYTES


def _codebook(dim, n):
    return tables.fib_codebook(dim, 4, n, 42, 512, 2, 4)


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("norm_format,order,n_codewords", [(L.NORM_FP16, L.ARGMIN_PAIRWISE, 32),
                                                          (L.NORM_F32, L.ARGMIN_SEQUENTIAL, 32),
                                                          (L.NORM_FP16, L.ARGMIN_SEQUENTIAL, 21),
                                                          (L.NORM_F32, L.ARGMIN_PAIRWISE, 6)])
def test_bytes_equal_the_oracle(oracle_mod, dim, norm_format, order, n_codewords):
    seed = 0x9E3779B97F4A7C15
    cb = _codebook(dim, n_codewords)
    prof = FibProfile(dim, None, cb, norm_format=norm_format, argmin_order=order, numerics=L.FIB_NUMERICS_BATCH,
                      hadamard_seed=seed)
    x = synthetic_kv(5000, dim, seed=dim + n_codewords)
    x[7] *= np.float32(1e-20) if norm_format == L.NORM_F32 else np.float32(1e-3)
    x[8] *= np.float32(1e12) if norm_format == L.NORM_F32 else np.float32(100.0)
    x[9, 1:] = 0.0                                       # one nonzero coordinate
    got = np.frombuffer(prof.encode_batch_compact(x), np.uint8)[H:].reshape(5000, -1)
    st, want, _, _ = oracle_mod.fib_encode_hadamard(x, seed, cb, norm_format=norm_format, argmin_order=order, nthreads=4)
    assert st == 0 and got.shape == want.shape
    assert np.array_equal(got, want), f"{np.count_nonzero((got != want).any(1))} records differ"


@pytest.mark.parametrize("dim", [64, 128])
def test_ragged_batches_in_one_launch(oracle_mod, dim):
    """Batches that end inside a 128-vector tile; one launch over all of them."""
    seed, cb = 5, _codebook(dim, 32)
    prof = FibProfile(dim, None, cb, numerics=L.FIB_NUMERICS_BATCH, hadamard_seed=seed)
    nb, vpb = 5, 333
    x = synthetic_kv(nb * vpb, dim, seed=3).reshape(nb, vpb, dim)
    out = np.zeros((nb, H + vpb * prof.record_bytes), np.uint8)
    encode_batches_compact(prof, x.ctypes.data, nb, vpb, out.ctypes.data, out.size)
    for b in range(nb):
        st, want, _, _ = oracle_mod.fib_encode_hadamard(x[b], seed, cb)
        assert st == 0 and np.array_equal(out[b, H:].reshape(vpb, -1), want), b


@pytest.mark.parametrize("dim", [64, 128])
def test_blocks_placed_on_codeword_bisectors(oracle_mod, dim):
    """Rotated blocks constructed at (and a few units in the last place around) the midpoint of two
    codewords: the certified search cannot decide them, the warp tier must, with the reference's tie rule."""
    seed, cb = 11, _codebook(dim, 32)
    m = tables.hadamard_rotation_matrix(dim, seed)
    rng = np.random.default_rng(8)
    n = 4096
    a, b = rng.integers(0, 32, (n, dim // 4)), rng.integers(0, 32, (n, dim // 4))
    y = 0.5 * (cb[a].astype(np.float64) + cb[b].astype(np.float64))            # [n, B, 4]
    y += rng.choice([0.0, 1e-8, -1e-8, 3e-7], size=y.shape) * rng.standard_normal(y.shape)
    y = y.reshape(n, dim)
    x = (y @ m).astype(np.float32)                                              # x = M^T y
    for order in (L.ARGMIN_PAIRWISE, L.ARGMIN_SEQUENTIAL):
        prof = FibProfile(dim, None, cb, argmin_order=order, numerics=L.FIB_NUMERICS_BATCH, hadamard_seed=seed)
        got = np.frombuffer(prof.encode_batch_compact(x), np.uint8)[H:].reshape(n, -1)
        st, want, _, _ = oracle_mod.fib_encode_hadamard(x, seed, cb, argmin_order=order, nthreads=4)
        assert st == 0 and np.array_equal(got, want)


def test_batch_size_threshold_and_errors(oracle_mod):
    """AUTO numerics: the stored matrix below 16 vectors (single-vector numerics below 4), the transform
    from 16 on, as the reference's `gpu` build decides; per-vector errors as in the dense encoder."""
    dim, seed, cb = 64, 77, _codebook(64, 32)
    rot = tables.haar_rotation(dim, 42)
    prof = FibProfile(dim, rot, cb, hadamard_seed=seed)
    x = synthetic_kv(64, dim, seed=1)
    for n in (3, 15):
        got = np.frombuffer(prof.encode_batch_compact(x[:n]), np.uint8)[H:].reshape(n, -1)
        st, want, _, _ = oracle_mod.fib_encode(x[:n], rot, cb)
        assert st == 0 and np.array_equal(got, want), n
    for n in (16, 64):
        got = np.frombuffer(prof.encode_batch_compact(x[:n]), np.uint8)[H:].reshape(n, -1)
        st, want, _, _ = oracle_mod.fib_encode_hadamard(x[:n], seed, cb)
        assert st == 0 and np.array_equal(got, want), n
    st, dense, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert not np.array_equal(dense, want)                # a different rotation: different indices
    for bad_row, value, code in ((20, np.nan, L.VEC_NONFINITE_INPUT), (33, 0.0, L.VEC_ZERO_NORM),
                                 (41, 3e4, L.VEC_NORM_RANGE)):
        xb = x.copy()
        xb[bad_row] = value
        st, _, ocode, oidx = oracle_mod.fib_encode_hadamard(xb, seed, cb)
        assert (ocode, oidx) == (code, bad_row)
        with pytest.raises(L.PkvError) as e:
            prof.encode_batch_compact(xb)
        assert (e.value.status, e.value.vector_index) == (code, bad_row)
    with pytest.raises(L.PkvError):
        FibProfile(dim, rot, cb, hadamard_seed=seed, numerics=L.FIB_NUMERICS_SINGLE)


@pytest.mark.parametrize("dim", [64, 128])
def test_decode_inverts_the_transform_when_the_profile_holds_it(dim):
    cb = tables.fib_codebook(dim, seed=42)
    prof = FibProfile(dim, None, cb, numerics=L.FIB_NUMERICS_BATCH, hadamard_seed=9)
    x = synthetic_kv(2048, dim, seed=2)
    def cosine(p_enc, p_dec):
        back = p_dec.decode_batch_compact(p_enc.encode_batch_compact(x))
        return float(((back * x).sum(1) / (np.linalg.norm(back, axis=1) * np.linalg.norm(x, axis=1))).mean())

    dense = FibProfile(dim, tables.haar_rotation(dim, 42), cb, numerics=L.FIB_NUMERICS_BATCH)
    c_h, c_d, c_mixed = cosine(prof, prof), cosine(dense, dense), cosine(prof, dense)
    # as good as the stored matrix at the same rate, and meaningless through a decoder that holds another matrix
    assert c_h > 0.8 and abs(c_h - c_d) < 0.03 and abs(c_mixed) < 0.1, (c_h, c_d, c_mixed)
