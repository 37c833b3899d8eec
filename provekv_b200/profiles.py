"""Codec profiles: the tables of one quantizer uploaded to the GPU, plus thin
methods over the C ABI (host-buffer "compact" calls and device-pointer calls).

A profile corresponds to one ``FibQuantizer`` (fib-quant/src/codec.rs:428-452) or
one ``TurboQuantizer`` (turbo-quant/src/turbo.rs:95-106) of the reference.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from . import tables


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _raise_vec(status: int, code: int, index: int):
    if status != L.OK:
        raise L.PkvError(status, L.status_string(status), index if status >= 16 else -1)


class _ProfileBase:
    _destroy = None
    handle = None

    def close(self):
        if self.handle is not None and L._lib is not None:
            getattr(L.lib(), self._destroy)(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class FibProfile(_ProfileBase):
    """fib-quant k=4 profile: dense rotation (dim x dim f64) + N x 4 f32 codebook."""
    _destroy = "pkv_fib_profile_destroy"

    def __init__(self, dim: int, rotation, codebook: np.ndarray, *,
                 norm_format: int = L.NORM_FP16, argmin_order: int = L.ARGMIN_PAIRWISE,
                 numerics: int = L.FIB_NUMERICS_AUTO, hadamard_seed: int | None = None):
        """hadamard_seed: encode batches with the f32 Walsh-Hadamard rotation of the reference's `gpu` build
        (fib-quant/src/codec.rs:612-656, gpu-backend/src/fallback.rs:12-88) seeded with it; `rotation` is then
        what the decoders invert and may be None (= the transform itself as a matrix).  Such payloads are not
        wire-compatible with pools encoded through the stored matrix."""
        self.dim = dim
        self.hadamard_seed = hadamard_seed
        if rotation is None:
            if hadamard_seed is None:
                raise ValueError("a rotation matrix is required unless hadamard_seed is given")
            rotation = tables.hadamard_rotation_matrix(dim, hadamard_seed)
        self.rotation = np.ascontiguousarray(rotation, dtype=np.float64).reshape(dim, dim)
        self.codebook = np.ascontiguousarray(codebook, dtype=np.float32)
        self.block_dim = self.codebook.shape[1]
        self.codebook_size = self.codebook.shape[0]
        cfg = L.FibConfigC(dim, self.block_dim, self.codebook_size, norm_format, argmin_order, numerics)
        self.norm_format, self.argmin_order, self.numerics = norm_format, argmin_order, numerics
        h = C.c_void_p()
        if hadamard_seed is None:
            L.check(L.lib().pkv_fib_profile_create(C.byref(cfg), _ptr(self.rotation), _ptr(self.codebook),
                                                   C.byref(h)))
        else:
            L.check(L.lib().pkv_fib_profile_create_hadamard(C.byref(cfg), C.c_uint64(hadamard_seed & (2 ** 64 - 1)),
                                                            _ptr(self.rotation), _ptr(self.codebook), C.byref(h)))
        self.handle = h
        self.record_bytes = L.lib().pkv_fib_record_bytes(h)

    @classmethod
    def from_seed(cls, dim: int, seed: int, *, k: int = 4, n: int = 32, training_samples: int = 2048,
                  restarts: int = 4, iterations: int = 8, **kw) -> "FibProfile":
        """Tables from this package's own seeded generators (not the Rust streams)."""
        return cls(dim, tables.haar_rotation(dim, seed),
                   tables.fib_codebook(dim, k, n, seed, training_samples, restarts, iterations), **kw)

    # -- host buffers, FB2 bytes (FibQuantAdapter::*_batch_compact) ------------
    def encode_batch_compact(self, vectors: np.ndarray) -> bytes:
        x = np.ascontiguousarray(vectors, dtype=np.float32).reshape(-1, self.dim)
        n = x.shape[0]
        out = np.empty(L.FB2_HEADER_BYTES + n * self.record_bytes, np.uint8)
        out_len, code, idx = C.c_int64(0), C.c_int32(0), C.c_int64(-1)
        st = L.lib().pkv_fib_encode_batch_compact(self.handle, _ptr(x), n, _ptr(out), out.size,
                                                  C.byref(out_len), C.byref(code), C.byref(idx))
        _raise_vec(st, code.value, idx.value)
        return out[:out_len.value].tobytes()

    def decode_batch_compact(self, payload: bytes) -> np.ndarray:
        buf = np.frombuffer(payload, np.uint8)
        n32 = C.c_uint32(0)
        L.check(L.lib().pkv_fb2_header_parse(self.handle, _ptr(buf), buf.size, C.byref(n32)))
        out = np.empty((n32.value, self.dim), np.float32)
        n, code, idx = C.c_int64(0), C.c_int32(0), C.c_int64(-1)
        st = L.lib().pkv_fib_decode_batch_compact(self.handle, _ptr(buf), buf.size, _ptr(out), out.size,
                                                  C.byref(n), C.byref(code), C.byref(idx))
        _raise_vec(st, code.value, idx.value)
        return out

    def decode_exact(self, records: bytes) -> np.ndarray:
        """FibQuantizer::decode (binary64 inverse rotation) of bare records -> [n, dim] f32."""
        buf = np.frombuffer(records, np.uint8)
        if buf.size % self.record_bytes:
            raise ValueError("records are not a whole number of vectors")
        n = buf.size // self.record_bytes
        out = np.empty((n, self.dim), np.float32)
        code, idx = C.c_int32(0), C.c_int64(-1)
        st = L.lib().pkv_fib_decode_exact(self.handle, _ptr(buf), n, _ptr(out), C.byref(code), C.byref(idx))
        _raise_vec(st, code.value, idx.value)
        return out

    def header(self, n_vectors: int) -> bytes:
        buf = (C.c_uint8 * L.FB2_HEADER_BYTES)()
        L.check(L.lib().pkv_fb2_header_write(self.handle, n_vectors, buf))
        return bytes(buf)

    # -- device pointers -------------------------------------------------------
    def encode_dev(self, x_ptr: int, layout: L.Layout, payload_ptr: int, payload_batch_stride: int,
                   err_ptr: int, stream: int = 0) -> None:
        L.check(L.lib().pkv_fib_encode_dev(self.handle, x_ptr, C.byref(layout), payload_ptr,
                                           payload_batch_stride, err_ptr, stream))

    def encode_dev_static(self, x_ptr: int, layout: L.Layout, payload_ptr: int,
                          payload_batch_stride: int, err_ptr: int, stream: int = 0) -> None:
        """encode_dev for callers that must not allocate device memory while encoding (HBM fully
        budgeted at start-up, allocator that may not be re-entered): the undecided-block list
        lives in a fixed 4 MiB array inside the library instead of the stream's memory pool.
        At most 2**20 vectors per call, batches of >= 4 vectors; calls on one device share the
        array, so do not let two of them overlap on the GPU."""
        L.check(L.lib().pkv_fib_encode_dev_static(self.handle, x_ptr, C.byref(layout), payload_ptr,
                                                  payload_batch_stride, err_ptr, stream))

    def decode_patch_dev(self, payload_ptr: int, payload_batch_stride: int, layout: L.Layout,
                         cache_ptr: int, err_ptr: int, stream: int = 0, dst_dtype: int = L.DST_F32) -> None:
        """dst_dtype: element type of the cache (L.DST_F32 / DST_F16 / DST_BF16); the 16-bit types
        are rounded to nearest-even in the store and need strides in multiples of 8 elements."""
        L.check(L.lib().pkv_fib_decode_patch_dev_as(self.handle, payload_ptr, payload_batch_stride,
                                                    C.byref(layout), cache_ptr, dst_dtype, err_ptr, stream))


    def decode_patch_dev_multi(self, payload_ptr: int, payload_batch_stride: int, layout: L.Layout,
                               cache_ptr: int, batch_offsets_ptr: int, err_ptr: int, stream: int = 0,
                               dst_dtype: int = L.DST_F32) -> None:
        """One launch over separately allocated cache tensors: batch b goes to
        cache_ptr + offsets[b] elements (device int64 table, non-negative multiples of 16 bytes)."""
        L.check(L.lib().pkv_fib_decode_patch_dev_multi(self.handle, payload_ptr, payload_batch_stride,
                                                       C.byref(layout), cache_ptr, batch_offsets_ptr,
                                                       dst_dtype, err_ptr, stream))


class TurboProfile(_ProfileBase):
    """turbo-quant profile: Rademacher signs, optional QJL matrix, angle LUT."""
    _destroy = "pkv_turbo_profile_destroy"

    def __init__(self, dim: int, bits: int, signs: np.ndarray, qjl: np.ndarray | None = None, *,
                 mode: int = L.TURBO_POLAR_WITH_QJL, radii_codec: int = L.RADII_F32, seed: int = 0,
                 cos_lut: np.ndarray | None = None, sin_lut: np.ndarray | None = None,
                 libm: int = L.LIBM_PORTABLE):
        """libm (BlockLogU8 radii only): L.LIBM_PORTABLE = correctly rounded logf / expf, the same bytes on
        every machine; L.LIBM_PLATFORM = this host's libm bit for bit, what the Rust reference writes here
        (the first such profile of a process scans every binary32 argument on the host: a few seconds)."""
        self.dim, self.bits, self.mode, self.radii_codec, self.seed = dim, bits, mode, radii_codec, seed
        self.libm = libm
        self.signs = np.ascontiguousarray(signs, dtype=np.float32)
        self.qjl = None if qjl is None else np.ascontiguousarray(qjl, dtype=np.float32)
        self.projections = 0 if self.qjl is None else self.qjl.shape[0]
        cfg = L.TurboConfigC(dim, bits, mode, self.projections, radii_codec, libm, seed)
        cl = None if cos_lut is None else np.ascontiguousarray(cos_lut, np.float32)
        sl = None if sin_lut is None else np.ascontiguousarray(sin_lut, np.float32)
        h = C.c_void_p()
        L.check(L.lib().pkv_turbo_profile_create(
            C.byref(cfg), _ptr(self.signs), None if self.qjl is None else _ptr(self.qjl),
            None if cl is None else _ptr(cl), None if sl is None else _ptr(sl), C.byref(h)))
        self.handle = h
        self.record_bytes = L.lib().pkv_turbo_record_bytes(h)

    @classmethod
    def from_seed(cls, dim: int, bits: int, projections: int, seed: int, *,
                  mode: int = L.TURBO_POLAR_WITH_QJL, radii_codec: int = L.RADII_F32,
                  sign_stream: str = "pcg64", libm: int = L.LIBM_PORTABLE) -> "TurboProfile":
        """sign_stream "chacha8": the Hadamard signs come from the reference's own ChaCha8 bool
        stream (tables.reference_hadamard_signs), which is all a polar-only profile needs from the
        seed; the QJL matrix is NumPy-seeded either way."""
        qjl = tables.qjl_matrix(dim, projections, seed) if mode == L.TURBO_POLAR_WITH_QJL else None
        if sign_stream not in ("pcg64", "chacha8"):
            raise ValueError("sign_stream must be 'pcg64' or 'chacha8'")
        signs = (tables.reference_hadamard_signs if sign_stream == "chacha8" else tables.rademacher_signs)(dim, seed)
        return cls(dim, bits, signs, qjl, mode=mode, radii_codec=radii_codec, seed=seed, libm=libm)

    def encode_batch_compact(self, vectors: np.ndarray) -> bytes:
        x = np.ascontiguousarray(vectors, dtype=np.float32).reshape(-1, self.dim)
        n = x.shape[0]
        out = np.empty(L.TQB1_HEADER_BYTES + n * self.record_bytes, np.uint8)
        out_len, code, idx = C.c_int64(0), C.c_int32(0), C.c_int64(-1)
        st = L.lib().pkv_turbo_encode_batch_compact(self.handle, _ptr(x), n, _ptr(out), out.size,
                                                    C.byref(out_len), C.byref(code), C.byref(idx))
        _raise_vec(st, code.value, idx.value)
        return out[:out_len.value].tobytes()

    def decode_batch_compact(self, payload: bytes) -> np.ndarray:
        buf = np.frombuffer(payload, np.uint8)
        n32 = C.c_uint32(0)
        L.check(L.lib().pkv_tqb1_header_parse(self.handle, _ptr(buf), buf.size, C.byref(n32)))
        out = np.empty((n32.value, self.dim), np.float32)
        n, code, idx = C.c_int64(0), C.c_int32(0), C.c_int64(-1)
        st = L.lib().pkv_turbo_decode_batch_compact(self.handle, _ptr(buf), buf.size, _ptr(out),
                                                    out.size, C.byref(n), C.byref(code), C.byref(idx))
        _raise_vec(st, code.value, idx.value)
        return out

    def header(self, n_vectors: int) -> bytes:
        buf = (C.c_uint8 * L.TQB1_HEADER_BYTES)()
        L.check(L.lib().pkv_tqb1_header_write(self.handle, n_vectors, buf))
        return bytes(buf)

    def encode_dev(self, x_ptr: int, layout: L.Layout, payload_ptr: int, payload_batch_stride: int,
                   err_ptr: int, stream: int = 0) -> None:
        L.check(L.lib().pkv_turbo_encode_dev(self.handle, x_ptr, C.byref(layout), payload_ptr,
                                             payload_batch_stride, err_ptr, stream))

    def decode_patch_dev(self, payload_ptr: int, payload_batch_stride: int, layout: L.Layout,
                         cache_ptr: int, err_ptr: int, stream: int = 0, dst_dtype: int = L.DST_F32) -> None:
        L.check(L.lib().pkv_turbo_decode_patch_dev_as(self.handle, payload_ptr, payload_batch_stride,
                                                      C.byref(layout), cache_ptr, dst_dtype, err_ptr, stream))


    def decode_patch_dev_multi(self, payload_ptr: int, payload_batch_stride: int, layout: L.Layout,
                               cache_ptr: int, batch_offsets_ptr: int, err_ptr: int, stream: int = 0,
                               dst_dtype: int = L.DST_F32) -> None:
        L.check(L.lib().pkv_turbo_decode_patch_dev_multi(self.handle, payload_ptr, payload_batch_stride,
                                                         C.byref(layout), cache_ptr, batch_offsets_ptr,
                                                         dst_dtype, err_ptr, stream))


    def prepare_query(self, query) -> tuple[np.ndarray, np.ndarray]:
        """TurboQuantizer::prepare_query (turbo-quant/src/turbo.rs:322-337) on the host, in the
        reference's binary32 operation order: (rotated, projected) = (FastHadamardRotation::apply(q),
        G q).  `projected` is empty for a polar-only profile."""
        q = np.ascontiguousarray(query, dtype=np.float32).reshape(-1)
        if q.size != self.dim:
            raise ValueError(f"query has {q.size} values, expected {self.dim}")
        if not np.all(np.isfinite(q)):
            raise ValueError("query is not finite")
        v = (q * self.signs).astype(np.float32)
        step = 1
        while step < self.dim:  # butterflies (a, b) -> (a + b, a - b) on (i, i + step), rotation.rs:379-398
            w = v.reshape(-1, 2, step)
            v = np.stack([w[:, 0, :] + w[:, 1, :], w[:, 0, :] - w[:, 1, :]], axis=1).astype(np.float32).reshape(-1)
            step *= 2
        rotated = (v * (np.float32(1.0) / np.sqrt(np.float32(self.dim)))).astype(np.float32)
        if self.qjl is None:
            return rotated, np.zeros(0, np.float32)
        prod = (self.qjl * q[None, :]).astype(np.float32)  # g * q, each rounded
        acc = np.zeros(self.qjl.shape[0], np.float32)
        for k in range(self.dim):  # summed in order, qjl.rs:277
            acc = (acc + prod[:, k]).astype(np.float32)
        return rotated, acc

    def score_dev(self, payload_ptr: int, payload_batch_stride: int, n_batches: int, vectors_per_batch: int,
                  rotated_ptr: int, projected_ptr: int, scores_ptr: int, err_ptr: int, stream: int = 0) -> None:
        """Inner-product estimates of one prepared query against every record of the launch
        (TurboQuantizer::score_batch_prepared, turbo.rs:340-381), read straight from the records."""
        L.check(L.lib().pkv_turbo_score_dev(self.handle, payload_ptr, payload_batch_stride, n_batches,
                                            vectors_per_batch, rotated_ptr, projected_ptr, scores_ptr,
                                            err_ptr, stream))


    def score_queries_dev(self, payload_ptr: int, payload_batch_stride: int, n_batches: int, vectors_per_batch: int,
                          rotated_ptr: int, projected_ptr: int, n_queries: int, scores_ptr: int, err_ptr: int,
                          stream: int = 0) -> None:
        """score_dev for n_queries prepared queries ([n_queries][dim] / [n_queries][projections] on the device)
        in one pass over the records; scores are [n_queries][n_batches * vectors_per_batch]."""
        L.check(L.lib().pkv_turbo_score_queries_dev(self.handle, payload_ptr, payload_batch_stride, n_batches,
                                                    vectors_per_batch, rotated_ptr, projected_ptr, n_queries,
                                                    scores_ptr, err_ptr, stream))

    def prepare_queries_dev(self, queries_ptr: int, n_queries: int, rotated_ptr: int, projected_ptr: int,
                            err_ptr: int, stream: int = 0) -> None:
        """TurboQuantizer::prepare_query (turbo.rs:322-337) on the device for [n_queries][dim] f32 queries."""
        L.check(L.lib().pkv_turbo_prepare_queries_dev(self.handle, queries_ptr, n_queries, rotated_ptr,
                                                      projected_ptr, err_ptr, stream))


def read_error_word(err_ptr: int, stream: int = 0) -> None:
    """Synchronise the stream and raise PkvError if a kernel reported a vector."""
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = L.lib().pkv_error_word_read(err_ptr, stream, C.byref(code), C.byref(idx))
    if st != L.OK:
        raise L.PkvError(st, L.status_string(st), idx.value)


def _bulk(fn_name: str, profile, src_ptr: int, n_batches: int, vpb: int, dst_ptr: int, dst_capacity: int):
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = getattr(L.lib(), fn_name)(profile.handle, src_ptr, n_batches, vpb, dst_ptr, dst_capacity,
                                   C.byref(code), C.byref(idx))
    _raise_vec(st, code.value, idx.value)


def encode_batches_compact(profile, vectors_ptr: int, n_batches: int, vectors_per_batch: int,
                           out_ptr: int, out_capacity: int) -> None:
    """Host [n_batches][vpb][dim] f32 -> n_batches wire blobs (header + records) at out_ptr.

    One call per pool / shell build instead of one per (layer, K|V); pointers are raw host
    addresses (pinned memory gives full PCIe rate)."""
    kind = "turbo" if isinstance(profile, TurboProfile) else "fib"
    _bulk(f"pkv_{kind}_encode_batches_compact", profile, vectors_ptr, n_batches, vectors_per_batch,
          out_ptr, out_capacity)


def decode_batches_compact(profile, bytes_ptr: int, n_batches: int, vectors_per_batch: int,
                           out_ptr: int, out_capacity_floats: int) -> None:
    kind = "turbo" if isinstance(profile, TurboProfile) else "fib"
    _bulk(f"pkv_{kind}_decode_batches_compact", profile, bytes_ptr, n_batches, vectors_per_batch,
          out_ptr, out_capacity_floats)
