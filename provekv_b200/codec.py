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


class InvalidShape(ProveKvError):
    pass


class InvalidManifest(ProveKvError):
    pass


class InvalidReceipt(ProveKvError):
    pass


class CorruptPayload(ProveKvError):
    pass


class DimensionMismatch(ProveKvError):
    pass


class CompressionFailed(ProveKvError):
    pass


class DecompressionFailed(ProveKvError):
    pass


@dataclass(frozen=True)
class FibConfig:
    """proveKV/src/policy.rs:117-182."""
    k: int = 4
    n: int = 32
    training_samples: int = 2048
    lloyd_restarts: int = 4
    lloyd_iterations: int = 8

    def validate(self) -> None:
        """policy.rs:147-182, same order of checks and messages."""
        if self.k == 0:
            raise InvalidPolicy("fib k must be > 0")
        if self.n < 2:
            raise InvalidPolicy("fib N must be >= 2")
        if self.k > 256:
            raise InvalidPolicy("fib k must be <= 256")
        if self.n > 1_048_576:
            raise InvalidPolicy("fib N must be <= 1,048,576")
        if self.training_samples == 0:
            raise InvalidPolicy("fib training_samples must be > 0")
        if self.lloyd_restarts == 0:
            raise InvalidPolicy("fib lloyd_restarts must be > 0")
        if self.lloyd_iterations == 0:
            raise InvalidPolicy("fib lloyd_iterations must be > 0")

    def as_json(self) -> dict:
        """Fields in declaration order, as serde writes the struct."""
        return {"k": self.k, "n": self.n, "training_samples": self.training_samples,
                "lloyd_restarts": self.lloyd_restarts, "lloyd_iterations": self.lloyd_iterations}


@dataclass(frozen=True)
class TurboConfig:
    """proveKV/src/policy.rs:218-290; ``lossy_radii`` is RadiiCompression::Lossy."""
    bits: int = 4
    projections: int = 32
    lossy_radii: bool = False

    def validate(self) -> None:
        """policy.rs:264-277."""
        if self.bits < 2 or self.bits > 16:
            raise InvalidPolicy(f"turbo bits must be 2\u201316, got {self.bits}")
        if self.projections == 0:
            raise InvalidPolicy("turbo projections must be > 0")

    def expected_compression_ratio(self) -> float:
        """policy.rs:279-288."""
        return 32.0 if self.lossy_radii else 8.0

    def as_json(self) -> dict:
        """The unit variants of RadiiCompression serialise as their names (policy.rs:208-213)."""
        return {"bits": self.bits, "projections": self.projections,
                "radii_compression": "Lossy" if self.lossy_radii else "Lossless"}

    @classmethod
    def from_json(cls, obj: dict) -> "TurboConfig":
        """`radii_compression` defaults to Lossless when absent (policy.rs:226 `serde(default)`)."""
        rc = obj.get("radii_compression", "Lossless")
        if rc not in ("Lossless", "Lossy"):
            raise InvalidPolicy(f"unknown radii_compression: {rc}")
        return cls(int(obj["bits"]), int(obj["projections"]), rc == "Lossy")


@functools.lru_cache(maxsize=16)
def _fib_profile(dim, k, n, ts, restarts, iters, seed, numerics=L.FIB_NUMERICS_AUTO) -> FibProfile:
    return FibProfile.from_seed(dim, seed, k=k, n=n, training_samples=ts, restarts=restarts,
                                iterations=iters, numerics=numerics)


# -- per-vector wire formats (host-side framing around the same records) --------------------------
FB1_MAGIC = b"FB1"       # fib-quant/src/codec.rs:20-21
FB1_HEADER_BYTES = 11    # magic, version, wire_index_bits, block_count u32, norm_len u16 (codec.rs:81-92)
TQW1_MAGIC = b"TQW1"     # turbo-quant/src/wire.rs:17
TQW1_HEADER_BYTES = 46   # wire.rs:74-88


def fb1_frame(record: bytes, wire_index_bits: int, block_count: int, norm_len: int) -> bytes:
    """FibCodeV1::to_compact_bytes (codec.rs:81-92): header, norm payload, packed indices."""
    return (FB1_MAGIC + bytes([1, wire_index_bits]) + int(block_count).to_bytes(4, "little") +
            int(norm_len).to_bytes(2, "little") + bytes(record))


def fb1_parse(blob: bytes, wire_index_bits: int, block_count: int, norm_len: int) -> bytes:
    """FibCodeV1::from_compact_bytes (codec.rs:100-152) -> the [norm][indices] record."""
    if len(blob) < FB1_HEADER_BYTES:
        raise DecompressionFailed(f"compact FibCodeV1 too short: {len(blob)} bytes (need >= 11)")
    if blob[0:3] != FB1_MAGIC:
        raise DecompressionFailed("compact FibCodeV1 bad magic")
    if blob[3] != 1:
        raise DecompressionFailed(f"compact FibCodeV1 version {blob[3]} not supported (need 1)")
    bits, blocks = blob[4], int.from_bytes(blob[5:9], "little")
    nlen = int.from_bytes(blob[9:11], "little")
    if len(blob) < FB1_HEADER_BYTES + nlen:
        raise DecompressionFailed("compact FibCodeV1 truncated")
    if len(blob) - FB1_HEADER_BYTES - nlen != (blocks * bits + 7) // 8:
        raise DecompressionFailed("compact FibCodeV1 indices: wrong packed length")
    if (bits, blocks, nlen) != (wire_index_bits, block_count, norm_len):
        raise DecompressionFailed("compact FibCodeV1 does not match the quantizer profile")
    return bytes(blob[FB1_HEADER_BYTES:])


def tqw1_frame(record: bytes, dim: int, polar_bits: int, projections: int, seed: int, with_qjl: bool) -> bytes:
    """TurboCodeWireV1::encode (wire.rs:44-96): f32 radii, packed angle indices, packed signs."""
    rotation_flag = 1 if dim & (dim - 1) == 0 else 0  # FastHadamard for power-of-two dims (wire.rs:583-589)
    head = (TQW1_MAGIC + (1).to_bytes(2, "little") + rotation_flag.to_bytes(2, "little") + bytes([1, 0]) +
            int(dim).to_bytes(4, "little") + bytes([polar_bits, 0, 0, 0]) + int(projections).to_bytes(4, "little") +
            int(seed).to_bytes(8, "little") + (dim // 2).to_bytes(4, "little") +
            (projections if with_qjl else 0).to_bytes(4, "little") + len(record).to_bytes(8, "little"))
    return head + bytes(record)


def tqw1_parse(blob: bytes, dim: int, polar_bits: int, projections: int, seed: int, with_qjl: bool) -> bytes:
    """TurboCodeWireV1::decode header checks (wire.rs:98-214) -> the vector's record."""
    if len(blob) < TQW1_HEADER_BYTES or blob[0:4] != TQW1_MAGIC:
        raise DecompressionFailed("wrong TurboQuant wire magic")
    u = lambda a, n: int.from_bytes(blob[a:a + n], "little")  # noqa: E731
    if u(4, 2) != 1:
        raise DecompressionFailed(f"unsupported TurboQuant wire version {u(4, 2)}")
    if u(6, 2) != (1 if dim & (dim - 1) == 0 else 0):
        raise DecompressionFailed("wire rotation flag does not match quantizer profile flag")
    if blob[8] != 1:
        raise DecompressionFailed(f"unsupported TurboQuant wire variant {blob[8]}")
    if blob[9] != 0 or blob[15:18] != b"\0\0\0":
        raise DecompressionFailed("nonzero TurboQuant wire reserved byte")
    if (u(10, 4), blob[14], u(18, 4)) != (dim, polar_bits, projections):
        raise DecompressionFailed("wire header does not match quantizer profile")
    if u(22, 8) != seed:
        raise DecompressionFailed(f"wire seed {u(22, 8)} does not match quantizer profile seed {seed}")
    if u(30, 4) != dim // 2:
        raise DecompressionFailed("wire polar block count does not match dimension")
    if u(34, 4) != (projections if with_qjl else 0):
        raise DecompressionFailed("wire sign count does not match expected")
    expect = 4 * (dim // 2) + ((dim // 2) * polar_bits + 7) // 8 + ((projections + 7) // 8 if with_qjl else 0)
    if u(38, 8) != expect or len(blob) != TQW1_HEADER_BYTES + expect:
        raise DecompressionFailed("TurboQuant wire payload length does not match expected")
    return bytes(blob[TQW1_HEADER_BYTES:])


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

    # -- per-vector payloads (FB1), codec.rs:581-667 ------------------------------------------
    def _wire_shape(self, prof: FibProfile):
        """(wire_index_bits, block_count, norm payload bytes) of the profile's codes."""
        return (max(1, (prof.codebook_size - 1).bit_length()), self._dim // self.k,
                2 if prof.norm_format == L.NORM_FP16 else 4)

    def _records(self, prof: FibProfile, x: np.ndarray) -> list[bytes]:
        fb2 = prof.encode_batch_compact(x)
        rec = prof.record_bytes
        bits, blocks, nlen = self._wire_shape(prof)
        return [fb1_frame(fb2[L.FB2_HEADER_BYTES + i * rec:L.FB2_HEADER_BYTES + (i + 1) * rec], bits, blocks, nlen)
                for i in range(x.shape[0])]

    def encode(self, vector, seed: int) -> bytes:
        """codec.rs:581-594: one vector, single-vector numerics, FB1 bytes (23 at d=64)."""
        x = _as_matrix([vector], self._dim, CompressionFailed)
        prof = _fib_profile(self._dim, self.k, self.n, self.training_samples, self.lloyd_restarts,
                            self.lloyd_iterations, seed, L.FIB_NUMERICS_SINGLE)
        try:
            return self._records(prof, x)[0]
        except L.PkvError as e:
            raise CompressionFailed(f"fib encode failed: {e}") from e

    def encode_batch(self, vectors, seed: int) -> list[bytes]:
        """codec.rs:596-610: FibQuantizer::encode_batch numerics, one FB1 payload per vector."""
        x = _as_matrix(vectors, self._dim, CompressionFailed)
        try:
            return self._records(self.build_quantizer(seed), x)
        except L.PkvError as e:
            raise CompressionFailed(f"fib encode_batch failed: {e}") from e

    def decode_batch(self, payloads, seed: int) -> np.ndarray:
        """codec.rs:640-667: FB1 payloads through decode_batch_fast -> [n, dim] f32.  (The JSON
        envelope of older pools is not read here.)"""
        prof = self.build_quantizer(seed)
        bits, blocks, nlen = self._wire_shape(prof)
        recs = [fb1_parse(bytes(p), bits, blocks, nlen) for p in payloads]
        try:
            return prof.decode_batch_compact(prof.header(len(recs)) + b"".join(recs))
        except L.PkvError as e:
            raise DecompressionFailed(f"fib decode_batch_fast failed: {e}") from e

    def decode(self, payload, seed: int) -> np.ndarray:
        """codec.rs:612-638: one FB1 payload through FibQuantizer::decode, i.e. the binary64 inverse
        rotation (not the batched f32 arithmetic of decode_batch)."""
        prof = self.build_quantizer(seed)
        bits, blocks, nlen = self._wire_shape(prof)
        rec = fb1_parse(bytes(payload), bits, blocks, nlen)
        try:
            return prof.decode_exact(rec)[0]
        except L.PkvError as e:
            raise DecompressionFailed(f"fib decode failed: {e}") from e


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

    # -- per-vector payloads (TQW1, always f32 radii), codec.rs:341-412 --------------------------
    def encode_batch(self, vectors, seed: int) -> list[bytes]:
        x = _as_matrix(vectors, self._dim, CompressionFailed)
        prof = _turbo_profile(self._dim, self.bits, self.projections, False, seed)
        try:
            tqb = prof.encode_batch_compact(x)
        except L.PkvError as e:
            raise CompressionFailed(f"turbo encode failed: {e}") from e
        rec = prof.record_bytes
        return [tqw1_frame(tqb[L.TQB1_HEADER_BYTES + i * rec:L.TQB1_HEADER_BYTES + (i + 1) * rec], self._dim,
                           self.bits - 1, self.projections, seed, True) for i in range(x.shape[0])]

    def encode(self, vector, seed: int) -> bytes:
        """codec.rs:341-368: TurboQuantizer::encode + TurboCodeWireV1::encode (46-byte header)."""
        return self.encode_batch([vector], seed)[0]

    def decode_batch(self, payloads, seed: int) -> np.ndarray:
        prof = _turbo_profile(self._dim, self.bits, self.projections, False, seed)
        recs = [tqw1_parse(bytes(p), self._dim, self.bits - 1, self.projections, seed, True) for p in payloads]
        try:
            return prof.decode_batch_compact(prof.header(len(recs)) + b"".join(recs))
        except L.PkvError as e:
            raise DecompressionFailed(f"turbo decode failed: {e}") from e

    def decode(self, payload, seed: int) -> np.ndarray:
        """codec.rs:370-412: the polar reconstruction of one TQW1 payload (the QJL signs are not
        invertible and are ignored, as in the reference)."""
        return self.decode_batch([payload], seed)[0]

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
