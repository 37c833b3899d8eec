"""The random streams the reference derives its tables from, restated from the published algorithms.

The reference seeds `rand_chacha::ChaCha8Rng` (0.3.1) with `seed_from_u64` and draws from `rand` 0.8.6
and `rand_distr` 0.4.3 (Cargo.lock): `gen::<bool>()` for the Hadamard signs, `StandardNormal` for the
QJL matrix and the Gaussian matrix behind the rotation, `Gamma` and `StandardNormal` for the training
samples of the codebook.  None of those crates is present here, so this module restates the
algorithms they document:

  * ChaCha8 block function, word stream, `seed_from_u64` (PCG32 key expansion): `tables.chacha_block`,
    checked against the published zero-key keystreams.
  * 64-bit draws: two consecutive 32-bit words of the stream, low word first.
  * uniform f64 in [0, 1): the top 53 bits times 2^-53; in the open interval (0, 1): the top 52 bits
    as the fraction of a float in [1, 2), minus (1 - 2^-53).
  * standard normal: the 256-layer ziggurat of Marsaglia and Tsang (2000) as Doornik (2005) corrects
    it: one 64-bit draw gives the layer (low 8 bits) and a uniform in [-1, 1) (top 52 bits); accept when
    |u x_i| < x_{i+1}; layer 0 falls back to the tail algorithm; otherwise accept against the density.
    The layer table is *computed* here from r = 3.654152885361008796 by the defining recurrence; the
    crates ship a printed copy of the same table, which may differ from this one in the last place.
  * gamma (shape a, scale 1): Marsaglia and Tsang's squeeze method for a >= 1, the boost u^(1/a) for
    a < 1.  (a = 1 is an exponential, which the crates draw from a second ziggurat: not restated.)
  * Householder QR in the formulation nalgebra documents (reflection axis x + sign(x_0) |x| e_0 scaled to
    unit length, diagonal of R kept as -sign(x_0) |x|, Q accumulated from the identity in reverse
    order).  The dot products here are NumPy's, whose summation order differs from nalgebra's.

No output of the Rust crates exists in this repository to compare with: everything above is
**unverified against the crates** beyond the ChaCha block function, and a table built here is only a
candidate for the table the reference builds from the same seed.  The codec's bit-exactness is defined
given equal tables and does not depend on this module.
"""
from __future__ import annotations

import math

import numpy as np

from .tables import chacha_block, seed_from_u64_key

_M64 = (1 << 64) - 1
ZIG_NORM_R = 3.654152885361008796
ZIG_LAYERS = 256


class ChaCha8Stream:
    """`ChaCha8Rng::seed_from_u64(seed)`: 32-bit words in block order; 64-bit draws pair them low word first."""

    def __init__(self, seed: int):
        self._key = seed_from_u64_key(seed & _M64)
        self._counter = 0
        self._buf: list = []
        self._pos = 0

    def next_u32(self) -> int:
        if self._pos >= len(self._buf):
            self._buf = chacha_block(self._key, self._counter, 0, 8)
            self._counter += 1
            self._pos = 0
        w = self._buf[self._pos]
        self._pos += 1
        return w

    def next_u64(self) -> int:
        lo = self.next_u32()
        return lo | (self.next_u32() << 32)

    def gen_bool(self) -> bool:
        """`Standard` for bool: the top bit of a 32-bit draw."""
        return bool(self.next_u32() >> 31)

    def gen_f64(self) -> float:
        """`Standard` for f64: 53 random bits scaled into [0, 1)."""
        return (self.next_u64() >> 11) * 2.0 ** -53

    def open01(self) -> float:
        """`Open01` for f64: 52 random bits as the fraction of a float in [1, 2), shifted into (0, 1)."""
        return _float_from_fraction(self.next_u64() >> 12, 0) - (1.0 - 2.0 ** -53)


def _float_from_fraction(frac52: int, exponent: int) -> float:
    """The binary64 number 2^exponent * (1 + frac52 / 2^52)."""
    return math.ldexp(1.0 + frac52 * 2.0 ** -52, exponent)


def _density(x: float) -> float:
    return math.exp(-x * x / 2.0)


def ziggurat_normal_tables():
    """x_0 .. x_256 and f(x_i) for 256 layers of equal area v: x_1 = r, x_0 = v / f(r) (the base layer's
    rectangle stands in for its tail), x_{i+1} = f^-1(v / x_i + f(x_i)), x_256 = 0."""
    r = ZIG_NORM_R
    v = r * _density(r) + math.sqrt(math.pi / 2.0) * math.erfc(r / math.sqrt(2.0))
    x = [v / _density(r), r]
    for _ in range(2, ZIG_LAYERS):
        x.append(math.sqrt(-2.0 * math.log(v / x[-1] + _density(x[-1]))))
    x.append(0.0)
    return x, [_density(t) for t in x], v


_ZIG_X, _ZIG_F, _ZIG_V = ziggurat_normal_tables()


def standard_normal(rng: ChaCha8Stream) -> float:
    """One N(0, 1) draw (f64)."""
    while True:
        bits = rng.next_u64()
        i = bits & 0xFF
        u = _float_from_fraction(bits >> 12, 1) - (3.0 - 2.0 ** -53)   # [2, 4) shifted to [-1, 1)
        x = u * _ZIG_X[i]
        if abs(x) < _ZIG_X[i + 1]:
            return x
        if i == 0:
            # tail beyond r: x = -ln(U1) / r, accept when -2 ln(U2) >= x^2
            while True:
                tx = math.log(rng.open01()) / ZIG_NORM_R
                ty = math.log(rng.open01())
                if -2.0 * ty >= tx * tx:
                    break
            return tx - ZIG_NORM_R if u < 0.0 else ZIG_NORM_R - tx
        if _ZIG_F[i + 1] + (_ZIG_F[i] - _ZIG_F[i + 1]) * rng.gen_f64() < _density(x):
            return x


def standard_normal_f32(rng: ChaCha8Stream) -> np.float32:
    """The f32 draw is the f64 draw rounded."""
    return np.float32(standard_normal(rng))


def gamma(rng: ChaCha8Stream, shape: float) -> float:
    """Gamma(shape, 1)."""
    if shape <= 0.0 or not math.isfinite(shape):
        raise ValueError("gamma shape must be positive and finite")
    if shape == 1.0:
        raise NotImplementedError("shape 1 is an exponential, drawn from a ziggurat that is not restated here")
    if shape < 1.0:
        inv = 1.0 / shape
        return _gamma_large(rng, shape + 1.0) * rng.open01() ** inv
    return _gamma_large(rng, shape)


def _gamma_large(rng: ChaCha8Stream, shape: float) -> float:
    d = shape - 1.0 / 3.0
    c = 1.0 / math.sqrt(9.0 * d)
    while True:
        x = standard_normal(rng)
        v_cbrt = 1.0 + c * x
        if v_cbrt <= 0.0:
            continue
        v = v_cbrt * v_cbrt * v_cbrt
        u = rng.open01()
        x_sqr = x * x
        if u < 1.0 - 0.0331 * x_sqr * x_sqr or math.log(u) < 0.5 * x_sqr + d * (1.0 - v + math.log(v)):
            return d * v


def unit_sphere(rng: ChaCha8Stream, k: int) -> list:
    """fib-quant/src/spherical_beta.rs:92-112."""
    while True:
        values = [standard_normal(rng) for _ in range(k)]
        norm_sq = 0.0
        for t in values:
            norm_sq += t * t
        if norm_sq > 0.0 and math.isfinite(norm_sq):
            norm = math.sqrt(norm_sq)
            return [t / norm for t in values]


def spherical_beta_sample(rng: ChaCha8Stream, d: int, k: int) -> list:
    """fib-quant/src/spherical_beta.rs:58-68,114-126: squared radius Beta(k/2, (d-k)/2) from two gamma
    draws, then a direction."""
    if k == d:
        return unit_sphere(rng, k)
    a = gamma(rng, k / 2.0)
    b = gamma(rng, (d - k) / 2.0)
    r = math.sqrt(a / (a + b))
    return [r * t for t in unit_sphere(rng, k)]


def training_samples(d: int, k: int, count: int, codebook_seed: int) -> np.ndarray:
    """fib-quant/src/lloyd.rs:184-196 for the canonical spherical-Beta source."""
    rng = ChaCha8Stream(codebook_seed ^ 0x465155414E54)
    return np.array([spherical_beta_sample(rng, d, k) for _ in range(count)], dtype=np.float64)


def qjl_matrix(dim: int, projections: int, quantizer_seed: int) -> np.ndarray:
    """turbo-quant/src/qjl.rs:341-352 behind turbo.rs:167: projections x dim f32, row-major."""
    rng = ChaCha8Stream((quantizer_seed + 0xCAFEBABE00000001 + 0xDEADBEEF12345678) & _M64)
    return np.array([standard_normal_f32(rng) for _ in range(projections * dim)], dtype=np.float32).reshape(projections, dim)


def householder_qr(a: np.ndarray):
    """Q (n x n) and the diagonal kept for R of a square matrix, by Householder reflections in the
    formulation described in the module header."""
    a = np.array(a, dtype=np.float64, order="F")
    n = a.shape[0]
    diag = np.zeros(n)
    for j in range(n):
        axis = a[j:, j]
        sq = float(axis @ axis)
        norm = math.sqrt(sq)
        sign = math.copysign(1.0, axis[0])
        signed_norm = sign * norm
        factor = (sq + abs(axis[0]) * norm) * 2.0
        axis[0] += signed_norm
        if factor != 0.0:
            axis /= math.sqrt(factor)
            diag[j] = -signed_norm
            s = math.copysign(1.0, diag[j])
            for c in range(j + 1, n):
                col = a[j:, c]
                f = float(axis @ col) * (s * -2.0)
                col[:] = f * axis + s * col
        else:
            diag[j] = signed_norm
    q = np.eye(n)
    for j in range(n - 1, -1, -1):
        axis = a[j:, j]
        s = math.copysign(1.0, diag[j])
        for c in range(j, n):
            col = q[j:, c]
            f = float(axis @ col) * (s * -2.0)
            col[:] = f * axis + s * col
    return q, diag


def haar_rotation(dim: int, seed: int) -> np.ndarray:
    """fib-quant/src/rotation.rs:36-57: dim^2 normal draws fill the matrix column by column, QR, and the
    columns of Q whose R diagonal is negative change sign; row-major Q."""
    rng = ChaCha8Stream(seed)
    data = [standard_normal(rng) for _ in range(dim * dim)]
    m = np.array(data, dtype=np.float64).reshape(dim, dim).T      # from_vec is column-major
    q, diag = householder_qr(m)
    # Recent nalgebra versions report the diagonal of R by magnitude, so the reference's sign pass finds
    # nothing to flip; with a signed diagonal the columns with diag < 0 would change sign instead.
    r_diag = np.abs(diag)
    for j in range(dim):
        if r_diag[j] < 0.0:
            q[:, j] *= -1.0
    return np.ascontiguousarray(q)
