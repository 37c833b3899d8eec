"""The restated random streams (ChaCha8 word pairing, ziggurat normal, gamma, Householder QR): internal
consistency and distribution checks.  Nothing here can compare with the Rust crates' output, which is
not available; the module says so."""
import math

import numpy as np
import pytest

from provekv_b200 import rust_streams as R
from provekv_b200 import tables


def test_word_pairing_and_uniforms():
    words = tables.chacha8_next_u32(77, 40)
    rng = R.ChaCha8Stream(77)
    assert [rng.next_u32() for _ in range(3)] == words[:3]
    assert rng.next_u64() == words[3] | (words[4] << 32)
    assert rng.gen_bool() == bool(words[5] >> 31)
    u = rng.gen_f64()
    assert u == ((words[6] | (words[7] << 32)) >> 11) * 2.0 ** -53 and 0.0 <= u < 1.0
    o = rng.open01()
    assert 0.0 < o < 1.0
    # the extremes of the open interval: all-zero and all-one fractions
    assert R._float_from_fraction(0, 0) - (1.0 - 2.0 ** -53) == 2.0 ** -53
    assert R._float_from_fraction((1 << 52) - 1, 0) - (1.0 - 2.0 ** -53) == 1.0 - 2.0 ** -53
    assert R._float_from_fraction(0, 1) - (3.0 - 2.0 ** -53) == -1.0 + 2.0 ** -53 or \
        R._float_from_fraction(0, 1) - (3.0 - 2.0 ** -53) == -1.0


def test_ziggurat_layers_have_equal_area():
    x, f, v = R.ziggurat_normal_tables()
    assert len(x) == len(f) == 257 and x[1] == R.ZIG_NORM_R and x[256] == 0.0 and f[256] == 1.0
    assert all(a > b for a, b in zip(x[1:], x[2:]))
    assert abs(x[0] * f[1] - v) < 1e-15                       # base strip: rectangle standing in for strip + tail
    for i in range(1, 255):
        assert abs(x[i] * (f[i + 1] - f[i]) - v) < 1e-13      # x_i (f(x_{i+1}) - f(x_i)) = v
    # the topmost strip closes at the mode to within the accuracy r was published with
    assert abs(x[255] * (1.0 - f[255]) - v) < 1e-9
    assert abs(v - 0.00492867323399) < 1e-13


def test_normal_draws_are_standard_normal():
    from scipy import stats
    rng = R.ChaCha8Stream(2024)
    z = np.array([R.standard_normal(rng) for _ in range(200_000)])
    assert abs(z.mean()) < 0.01 and abs(z.var() - 1.0) < 0.01
    assert abs(stats.kurtosis(z)) < 0.05 and abs(stats.skew(z)) < 0.02
    assert stats.kstest(z, "norm").pvalue > 1e-3
    tail = np.mean(np.abs(z) > R.ZIG_NORM_R)
    assert 0.5 * 2.58e-4 < tail < 2.0 * 2.58e-4               # 2 (1 - Phi(r))
    again = R.ChaCha8Stream(2024)
    assert [R.standard_normal(again) for _ in range(100)] == list(z[:100])
    assert R.standard_normal_f32(R.ChaCha8Stream(2024)) == np.float32(z[0])


@pytest.mark.parametrize("shape", [0.5, 2.0, 30.0, 62.0])
def test_gamma_moments(shape):
    rng = R.ChaCha8Stream(int(shape * 10))
    g = np.array([R.gamma(rng, shape) for _ in range(40_000)])
    assert (g > 0).all()
    assert abs(g.mean() / shape - 1.0) < 0.03 and abs(g.var() / shape - 1.0) < 0.08
    with pytest.raises(NotImplementedError):
        R.gamma(rng, 1.0)


def test_training_samples_follow_the_block_law():
    d, k = 64, 4
    s = R.training_samples(d, k, 4000, 42)
    assert s.shape == (4000, k)
    r2 = (s * s).sum(axis=1)
    assert (r2 < 1.0).all() and abs(r2.mean() - k / d) < 0.004      # E |block|^2 = k / d
    assert np.abs(s.mean(axis=0)).max() < 0.01
    assert np.array_equal(s[:5], R.training_samples(d, k, 5, 42))


def test_householder_qr_and_rotation():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((24, 24))
    q, diag = R.householder_qr(a)
    assert np.abs(q.T @ q - np.eye(24)).max() < 1e-13
    r = q.T @ a
    assert np.abs(np.tril(r, -1)).max() < 1e-12 and np.allclose(np.abs(np.diag(r)), np.abs(diag), atol=1e-12)
    rot = R.haar_rotation(16, 5)
    assert rot.shape == (16, 16) and np.abs(rot @ rot.T - np.eye(16)).max() < 1e-13
    assert np.array_equal(rot, R.haar_rotation(16, 5)) and not np.array_equal(rot, R.haar_rotation(16, 6))


def test_qjl_matrix_from_the_stream():
    g = R.qjl_matrix(64, 32, 42)
    assert g.shape == (32, 64) and g.dtype == np.float32
    assert abs(float(g.mean())) < 0.08 and abs(float(g.var()) - 1.0) < 0.1
    first = R.standard_normal_f32(R.ChaCha8Stream((42 + 0xCAFEBABE00000001 + 0xDEADBEEF12345678) & (2 ** 64 - 1)))
    assert g[0, 0] == first
