"""Seeded generators for the tables the codec kernels take as inputs.

The reference derives its tables from a seed with ``rand_chacha`` (ChaCha8),
``rand_distr`` (ziggurat normal, gamma), ``nalgebra`` (Householder QR) and
``statrs`` (inverse CDFs).  Apart from `reference_hadamard_signs` (the ChaCha8
bool stream, restated below) those streams are not reproduced here: the
generators follow the same *algorithms* with NumPy's PCG64 as the random
source, so a table built here is a valid table of the same distribution but is
not the table the Rust crate builds for the same seed.  Bit-exactness of the
codec is defined given equal tables; tables are plain arrays that can also be
loaded from a dump of the Rust side.  `rust_streams.py` restates the crates'
own streams (ziggurat normal, gamma, Householder QR on ChaCha8) as candidates
for the reference's tables, unverified against the crates.

Reference algorithms followed:
  * Haar rotation        fib-quant/src/rotation.rs:24-58
  * Lloyd-Max codebook   fib-quant/src/codebook.rs:158-203, lloyd.rs:105-317,
                         directions.rs:38-114, spherical_beta.rs:6-139
  * Rademacher signs     turbo-quant/src/rotation.rs:143-157
  * QJL Gaussian matrix  turbo-quant/src/qjl.rs:341-352
"""
from __future__ import annotations

import functools

import numpy as np

_MASK64 = (1 << 64) - 1


_M64 = (1 << 64) - 1


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed & _MASK64))


def haar_rotation(dim: int, seed: int) -> np.ndarray:
    """dim x dim orthogonal f64 matrix, row-major.

    Gaussian matrix filled column-major (``DMatrix::from_vec``), QR, then the
    columns of Q whose R diagonal is negative are flipped
    (fib-quant/src/rotation.rs:36-50).
    """
    if dim <= 0:
        raise ValueError("dim must be positive")
    data = _rng(seed).standard_normal(dim * dim)
    m = data.reshape((dim, dim), order="F")
    q, r = np.linalg.qr(m)
    flip = np.diag(r) < 0.0
    q = q.copy()
    q[:, flip] *= -1.0
    return np.ascontiguousarray(q, dtype=np.float64)


def lcg_hadamard_signs(dim: int, seed: int) -> np.ndarray:
    """gpu-backend/src/fallback.rs:76-88: one step of state = state * 6364136223846793005 + 1442695040888963407
    (mod 2^64) per coordinate; bit 32 of the state set -> +1, clear -> -1."""
    state, out = seed & _M64, np.empty(dim, np.float32)
    for i in range(dim):
        state = (state * 6364136223846793005 + 1442695040888963407) & _M64
        out[i] = 1.0 if (state >> 32) & 1 else -1.0
    return out


def hadamard_rotation_matrix(dim: int, seed: int) -> np.ndarray:
    """The transform of gpu-backend/src/fallback.rs:12-62 for a power-of-two dim as a dim x dim f64 matrix:
    M[r][j] = sign_r * (1 / sqrt(dim) in f32) * (-1)^popcount(r & j).  Orthogonal to f32 rounding of the
    scale; a profile whose decoders hold it inverts what the Hadamard encoder applied."""
    if dim & (dim - 1):
        raise ValueError("dim must be a power of two")
    scale = np.float32(1.0) / np.sqrt(np.float32(dim))
    signs = lcg_hadamard_signs(dim, seed).astype(np.float64) * float(scale)
    r = np.arange(dim)
    parity = np.array([[bin(a & b).count("1") & 1 for b in r] for a in r])
    return np.where(parity == 1, -1.0, 1.0) * signs[:, None]


def rademacher_signs(dim: int, seed: int) -> np.ndarray:
    """dim values of +-1.0 (f32); seed offset as turbo-quant/src/rotation.rs:152."""
    bits = _rng((seed + 0xA11CE55ED5A5EED5) & _MASK64).integers(0, 2, size=dim)
    return np.where(bits == 1, 1.0, -1.0).astype(np.float32)


# --- the reference's own random stream (rand_chacha 0.3.1 ChaCha8Rng, rand_core 0.6.4, rand 0.8) ----
# Restated from the published algorithms (the crates are not vendored with the reference): the ChaCha
# block function with 8 rounds, 64-bit block counter in words 12-13 and stream id 0 in words 14-15,
# output words consumed in order; SeedableRng::seed_from_u64 fills the 32-byte key from a PCG32
# sequence; Standard's bool is the top bit of next_u32().  The block function is checked against
# the published zero-key ChaCha8 and ChaCha20 keystreams (tests/test_oracle_pins.py); no output of
# the Rust crate for a given seed exists here to compare with, so seed-level equality with the
# crate is unverified.
_M32 = 0xFFFFFFFF


def _rotl32(x: int, n: int) -> int:
    return ((x << n) & _M32) | (x >> (32 - n))


def _quarter_round(s: list, a: int, b: int, c: int, d: int) -> None:
    s[a] = (s[a] + s[b]) & _M32
    s[d] = _rotl32(s[d] ^ s[a], 16)
    s[c] = (s[c] + s[d]) & _M32
    s[b] = _rotl32(s[b] ^ s[c], 12)
    s[a] = (s[a] + s[b]) & _M32
    s[d] = _rotl32(s[d] ^ s[a], 8)
    s[c] = (s[c] + s[d]) & _M32
    s[b] = _rotl32(s[b] ^ s[c], 7)


def chacha_block(key_words, counter: int, stream: int = 0, rounds: int = 8) -> list:
    """One 16-word ChaCha block (original variant: 64-bit counter, 64-bit stream id)."""
    init = [0x61707865, 0x3320646E, 0x79622D32, 0x6B206574, *key_words,
            counter & _M32, (counter >> 32) & _M32, stream & _M32, (stream >> 32) & _M32]
    s = list(init)
    for _ in range(rounds // 2):
        _quarter_round(s, 0, 4, 8, 12)
        _quarter_round(s, 1, 5, 9, 13)
        _quarter_round(s, 2, 6, 10, 14)
        _quarter_round(s, 3, 7, 11, 15)
        _quarter_round(s, 0, 5, 10, 15)
        _quarter_round(s, 1, 6, 11, 12)
        _quarter_round(s, 2, 7, 8, 13)
        _quarter_round(s, 3, 4, 9, 14)
    return [(a + b) & _M32 for a, b in zip(s, init)]


def seed_from_u64_key(state: int) -> list:
    """The eight key words SeedableRng::seed_from_u64 derives from a u64: PCG32 steps
    (multiplier 6364136223846793005, increment 11634580027462260723, XSH-RR output), the state
    advanced before each output."""
    words = []
    for _ in range(8):
        state = (state * 6364136223846793005 + 11634580027462260723) & _MASK64
        xorshifted = (((state >> 18) ^ state) >> 27) & _M32
        rot = state >> 59
        words.append(((xorshifted >> rot) | (xorshifted << ((32 - rot) & 31))) & _M32)
    return words


def chacha8_next_u32(seed: int, n: int) -> list:
    """The first n next_u32() outputs of ChaCha8Rng::seed_from_u64(seed)."""
    key, out, counter = seed_from_u64_key(seed & _MASK64), [], 0
    while len(out) < n:
        out.extend(chacha_block(key, counter, 0, 8))
        counter += 1
    return out[:n]


def reference_hadamard_signs(dim: int, seed: int) -> np.ndarray:
    """FastHadamardRotation::new (turbo-quant/src/rotation.rs:152-155) on the reference's own
    stream: ChaCha8Rng::seed_from_u64(seed + 0xA11CE55ED5A5EED5), one gen::<bool>() per
    coordinate, true -> +1.0."""
    words = chacha8_next_u32((seed + 0xA11CE55ED5A5EED5) & _MASK64, dim)
    return np.array([1.0 if w >> 31 else -1.0 for w in words], dtype=np.float32)


def qjl_matrix(dim: int, projections: int, seed: int) -> np.ndarray:
    """projections x dim N(0,1) f32, row-major.

    ``seed`` is the TurboQuantizer seed; the two offsets are
    turbo-quant/src/turbo.rs:167 and turbo-quant/src/qjl.rs:346.
    """
    s = (seed + 0xCAFEBABE00000001 + 0xDEADBEEF12345678) & _MASK64
    g = _rng(s).standard_normal(projections * dim).astype(np.float32)
    return np.ascontiguousarray(g.reshape(projections, dim))


# --- fib-quant codebook ------------------------------------------------------

def _roberts_phi(k: int) -> float:
    lo, hi = 1.0, 2.0
    for _ in range(128):
        mid = (lo + hi) / 2.0
        if mid ** (k + 1) - mid - 1.0 > 0.0:
            hi = mid
        else:
            lo = mid
    return (lo + hi) / 2.0


def _roberts_kronecker(k: int, n: int) -> np.ndarray:
    """fib-quant/src/directions.rs:38-74."""
    from scipy.stats import norm

    phi = _roberts_phi(k)
    out = np.empty((n, k))
    for idx in range(n):
        for j in range(1, k + 1):
            step = phi ** (-j)
            frac = min(max(((idx + 0.5) * step) % 1.0, 1.0e-12), 1.0 - 1.0e-12)
            out[idx, j - 1] = norm.ppf(frac)
        out[idx] /= np.sqrt(np.sum(out[idx] ** 2))
    return out


def _beta_d_k(d: int, k: int) -> float:
    """fib-quant/src/spherical_beta.rs:6-21."""
    if k == d:
        return 1.0
    return (k / (k + 2.0)) * ((d - k - 2.0) / 2.0) + 1.0


def _initial_codebook(d: int, k: int, n: int) -> np.ndarray:
    """Radial-angular initialisation, fib-quant/src/codebook.rs:158-181 (k >= 4)."""
    from scipy.stats import beta as beta_dist

    if k < 4:
        raise ValueError("only the k >= 4 (Roberts-Kronecker) path is implemented")
    dirs = _roberts_kronecker(k, n)
    out = np.empty((n, k))
    for idx in range(n):
        if k == d:
            radius = 1.0
        else:
            q = (idx + 1 - 0.5) / n
            radius = np.sqrt(min(max(beta_dist.ppf(q, k / 2.0, _beta_d_k(d, k)), 0.0), 1.0))
        out[idx] = radius * dirs[idx]
    return out


def _nearest(samples: np.ndarray, codebook: np.ndarray):
    d2 = ((samples[:, None, :] - codebook[None, :, :]) ** 2).sum(axis=2)
    idx = np.argmin(d2, axis=1)  # first minimum == strict '<' scan
    return idx, d2[np.arange(len(samples)), idx]


def _lloyd_step(codebook: np.ndarray, samples: np.ndarray) -> None:
    """One assign + update_centroids pass with the split-highest-distortion repair
    (fib-quant/src/lloyd.rs:215-317)."""
    n, k = codebook.shape
    assign, dist = _nearest(samples, codebook)
    counts = np.bincount(assign, minlength=n)
    distortion = np.bincount(assign, weights=dist, minlength=n)
    farthest = np.zeros((n, k))
    far_d = np.full(n, -1.0)
    for s, a, dd in zip(samples, assign, dist):
        if dd > far_d[a]:
            far_d[a] = dd
            farthest[a] = s
    sums = np.zeros((n, k))
    np.add.at(sums, assign, samples)
    nz = counts > 0
    codebook[nz] = sums[nz] / counts[nz, None]
    counts = counts.copy()
    for empty in np.flatnonzero(counts == 0):
        donors = np.flatnonzero(counts > 1)
        if donors.size == 0:
            raise RuntimeError("no donor cell")
        # Rust's max_by keeps the last of equal maxima
        best = donors[0]
        for c in donors[1:]:
            if distortion[c] >= distortion[best]:
                best = c
        residual = farthest[best] - codebook[best]
        rn = np.sqrt(np.sum(residual ** 2))
        if not np.isfinite(rn) or rn <= np.finfo(np.float64).eps:
            raise RuntimeError("donor residual has zero direction")
        direction = residual / rn
        centroid = codebook[best].copy()
        codebook[best] = centroid - 1.0e-6 * direction
        codebook[empty] = centroid + 1.0e-6 * direction
        counts[best] -= 1
        counts[empty] = 1
        distortion[best] = 0.0
        distortion[empty] = 0.0


@functools.lru_cache(maxsize=32)
def _fib_codebook_cached(dim, k, n, seed, training_samples, restarts, iterations) -> bytes:
    codebook_seed = (seed + 0x9E3779B97F4A7C15) & _MASK64  # fib-quant/src/profile.rs:161
    initial = _initial_codebook(dim, k, n)
    # training set: canonical spherical-Beta k-block source (lloyd.rs:184-195)
    rng = _rng(codebook_seed ^ 0x465155414E54)
    count = max(training_samples, n)
    if k == dim:
        g = rng.standard_normal((count, k))
        samples = g / np.sqrt((g ** 2).sum(axis=1, keepdims=True))
    else:
        a = rng.gamma(k / 2.0, 1.0, size=count)
        b = rng.gamma((dim - k) / 2.0, 1.0, size=count)
        r = np.sqrt(a / (a + b))
        g = rng.standard_normal((count, k))
        samples = r[:, None] * g / np.sqrt((g ** 2).sum(axis=1, keepdims=True))
    init_mse = float(_nearest(samples, initial)[1].mean())
    best, best_mse = initial.copy(), init_mse
    for restart in range(max(restarts, 1)):
        if restart == 0:
            cb = initial.copy()
        else:  # rotated_initial, lloyd.rs:197-213
            rot = haar_rotation(k, (codebook_seed + restart * 0x9E3779B9) & _MASK64)
            cb = initial @ rot.T
        for _ in range(iterations):
            _lloyd_step(cb, samples)
        mse = float(_nearest(samples, cb)[1].mean())
        if mse < best_mse:
            best, best_mse = cb.copy(), mse
    return np.ascontiguousarray(best, dtype=np.float32).tobytes()


def fib_codebook(dim: int, k: int = 4, n: int = 32, seed: int = 42, training_samples: int = 2048,
                 restarts: int = 4, iterations: int = 8) -> np.ndarray:
    """N x k f32 Lloyd-Max codebook for the k-block of a random unit vector in R^dim.

    Defaults are proveKV's ``FibConfig::default_k4_n32`` (proveKV/src/policy.rs:137-145).
    """
    raw = _fib_codebook_cached(dim, k, n, seed, training_samples, restarts, iterations)
    return np.frombuffer(raw, dtype=np.float32).reshape(n, k).copy()
