"""Host-side mirror of proveKV's codec plug-in surface (proveKV/src/codec.rs).

Same names, argument meaning and error behaviour as the reference's
``KVecCodec`` trait (codec.rs:8-66), ``FibQuantAdapter`` (codec.rs:423-569),
``TurboQuantAdapter`` (codec.rs:170-326) and ``create_codec`` (codec.rs:700-758),
with the arithmetic done by the CUDA library.  Adapters are stateless value
objects as in the reference; the seed is passed per call and the GPU profile
(tables) for a seed is cached.
"""
from __future__ import annotations

import functools
from dataclasses import dataclass

import numpy as np

from . import _lib as L
from .profiles import FibProfile, TurboProfile

# codec identifiers, proveKV/src/policy.rs:8-24,78-82
CODEC_FIB_K4_N32 = "fib_k4_n32"
CODEC_FIB_K4_N32_BATCHED = "fib_k4_n32_batched"
CODEC_TURBO_8BIT = "turbo_8bit"
CODEC_TURBO_8BIT_BATCHED = "turbo_8bit_batched"
CODEC_TURBO_8BIT_BATCHED_LOSSY = "turbo_8bit_batched_lossy"
CODEC_EXACT_FALLBACK = "exact_f32_fallback"


def turbo_batched_codec_id(bits: int, lossy_radii: bool) -> str:
    return f"turbo_{bits}bit_batched{'_lossy' if lossy_radii else ''}"


class ProveKvError(Exception):
    """Base of the errors below (proveKV/src/error.rs:5-59)."""


class InvalidPolicy(ProveKvError):
    pass


class CompressionFailed(ProveKvError):
    pass


class DecompressionFailed(ProveKvError):
    pass


@dataclass(frozen=True)
class FibConfig:
    """proveKV/src/policy.rs:117-145."""
    k: int = 4
    n: int = 32
    training_samples: int = 2048
    lloyd_restarts: int = 4
    lloyd_iterations: int = 8


@dataclass(frozen=True)
class TurboConfig:
    """proveKV/src/policy.rs:218-262; ``lossy_radii`` is RadiiCompression::Lossy."""
    bits: int = 4
    projections: int = 32
    lossy_radii: bool = False


@functools.lru_cache(maxsize=16)
def _fib_profile(dim, k, n, ts, restarts, iters, seed) -> FibProfile:
    return FibProfile.from_seed(dim, seed, k=k, n=n, training_samples=ts, restarts=restarts,
                                iterations=iters)


@functools.lru_cache(maxsize=16)
def _turbo_profile(dim, bits, projections, lossy, seed) -> TurboProfile:
    return TurboProfile.from_seed(dim, bits, projections, seed, mode=L.TURBO_POLAR_WITH_QJL,
                                  radii_codec=L.RADII_BLOCK_LOG_U8 if lossy else L.RADII_F32)


def _as_matrix(vectors, dim: int, exc) -> np.ndarray:
    if isinstance(vectors, np.ndarray) and vectors.ndim == 2:
        x = vectors
    else:
        rows = [np.asarray(v, dtype=np.float32) for v in vectors]
        for r in rows:
            if r.shape != (dim,):
                raise exc(f"input dimension {r.size}, expected {dim}")
        x = np.stack(rows) if rows else np.empty((0, dim), np.float32)
    if x.shape[1] != dim:
        raise exc(f"input dimension {x.shape[1]}, expected {dim}")
    return np.ascontiguousarray(x, dtype=np.float32)


class KVecCodec:
    """The reference's codec trait (codec.rs:8-66)."""

    def codec_id(self) -> str:
        raise NotImplementedError

    def dim(self) -> int:
        raise NotImplementedError

    def compression_ratio(self) -> float:
        raise NotImplementedError

    def is_gpu_accelerated(self) -> bool:
        return True

    def is_gpu_accelerated_for(self, n: int, d: int) -> bool:
        return self.is_gpu_accelerated()


class FibQuantAdapter(KVecCodec):
    def __init__(self, dim: int, k: int, n: int, training_samples: int, lloyd_restarts: int,
                 lloyd_iterations: int):
        if dim == 0:
            raise InvalidPolicy("fib dim must be > 0")
        if dim % k != 0:
            raise InvalidPolicy(f"fib ambient dim ({dim}) must be divisible by k ({k})")
        self._dim, self.k, self.n = dim, k, n
        self.training_samples, self.lloyd_restarts, self.lloyd_iterations = (
            training_samples, lloyd_restarts, lloyd_iterations)

    def codec_id(self) -> str:
        return CODEC_FIB_K4_N32

    def dim(self) -> int:
        return self._dim

    def compression_ratio(self) -> float:
        return 21.33

    def build_quantizer(self, seed: int) -> FibProfile:
        """codec.rs:471-499: the quantizer (tables) for a seed."""
        return _fib_profile(self._dim, self.k, self.n, self.training_samples, self.lloyd_restarts,
                            self.lloyd_iterations, seed)

    def encode_batch_compact(self, vectors, seed: int) -> bytes:
        """codec.rs:513-525 -> FB2 bytes."""
        x = _as_matrix(vectors, self._dim, CompressionFailed)
        try:
            return self.build_quantizer(seed).encode_batch_compact(x)
        except L.PkvError as e:
            raise CompressionFailed(f"fib encode_batch failed: {e}") from e

    def decode_batch_compact(self, payload: bytes, seed: int) -> np.ndarray:
        """codec.rs:530-569 (FB2 payloads) -> [n, dim] f32."""
        try:
            return self.build_quantizer(seed).decode_batch_compact(payload)
        except L.PkvError as e:
            raise DecompressionFailed(f"fib batched wire decode failed: {e}") from e


class TurboQuantAdapter(KVecCodec):
    def __init__(self, dim: int, bits: int, projections: int, lossy_radii: bool = False):
        if dim == 0:
            raise InvalidPolicy("turbo dim must be > 0")
        if dim % 2 != 0:
            raise InvalidPolicy(f"turbo requires even dimension, got {dim}")
        self._dim, self.bits, self.projections, self.lossy_radii = dim, bits, projections, lossy_radii

    @classmethod
    def with_radii_compression(cls, dim, bits, projections, lossy_radii) -> "TurboQuantAdapter":
        return cls(dim, bits, projections, lossy_radii)

    def codec_id(self) -> str:
        return CODEC_TURBO_8BIT

    def dim(self) -> int:
        return self._dim

    def compression_ratio(self) -> float:
        return 8.0

    def build_quantizer(self, seed: int) -> TurboProfile:
        return _turbo_profile(self._dim, self.bits, self.projections, self.lossy_radii, seed)

    def encode_batch_compact(self, vectors, seed: int) -> bytes:
        """codec.rs:248-291 -> TQB1 bytes."""
        x = _as_matrix(vectors, self._dim, CompressionFailed)
        try:
            return self.build_quantizer(seed).encode_batch_compact(x)
        except L.PkvError as e:
            raise CompressionFailed(f"turbo encode failed: {e}") from e

    def decode_batch_compact(self, payload: bytes, seed: int) -> np.ndarray:
        """codec.rs:295-326; the radii codec is taken from byte 15 of the header."""
        lossy = len(payload) > 15 and payload[15] == 1
        try:
            prof = _turbo_profile(self._dim, self.bits, self.projections, lossy, seed)
            return prof.decode_batch_compact(payload)
        except L.PkvError as e:
            raise DecompressionFailed(f"turbo batched wire decode failed: {e}") from e


def create_codec(codec_id: str, dim: int, fib_config: FibConfig | None = None,
                 turbo_config: TurboConfig | None = None) -> KVecCodec:
    """codec.rs:700-758."""
    if codec_id in (CODEC_FIB_K4_N32, CODEC_FIB_K4_N32_BATCHED):
        if fib_config is None:
            raise InvalidPolicy("fib codec requires fib_config")
        fc = fib_config
        return FibQuantAdapter(dim, fc.k, fc.n, fc.training_samples, fc.lloyd_restarts,
                               fc.lloyd_iterations)
    if codec_id in (CODEC_TURBO_8BIT, CODEC_TURBO_8BIT_BATCHED):
        if turbo_config is None:
            raise InvalidPolicy("turbo codec requires turbo_config")
        return TurboQuantAdapter(dim, turbo_config.bits, turbo_config.projections)
    raise InvalidPolicy(f"unknown codec id: {codec_id}")
