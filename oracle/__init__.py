"""ctypes access to the CPU oracle (oracle/pkv_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke`` and
by ``bench.py``'s CPU-baseline legs.  The shipped package never imports it.
PARITY UNPINNED: see the header of pkv_oracle.c.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_DIR, "libpkv_oracle.so")

LIBM_PLATFORM = 0
LIBM_PORTABLE = 1


def build() -> str:
    """Compile the oracle with gcc (oracle/Makefile)."""
    subprocess.run(["make", "-C", _DIR], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.pkvo_f16_bits_to_f32.restype = C.c_float
        _lib.pkvo_f32_to_f16_bits.restype = C.c_uint16
        _lib.pkvo_f32_to_f16_bits.argtypes = [C.c_float]
        _lib.pkvo_f16_bits_to_f32.argtypes = [C.c_uint16]
        for name in ("pkvo_atan2f", "pkvo_logf", "pkvo_expf"):
            getattr(_lib, name).restype = C.c_float
        _lib.pkvo_atan2f.argtypes = [C.c_float, C.c_float, C.c_int]
        _lib.pkvo_logf.argtypes = [C.c_float, C.c_int]
        _lib.pkvo_expf.argtypes = [C.c_float, C.c_int]
        _lib.pkvo_angle_bucket.restype = C.c_uint32
        _lib.pkvo_angle_bucket.argtypes = [C.c_float, C.c_uint32]
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fib_record_bytes(dim, k=4, n_codewords=32, norm_format=0) -> int:
    return lib().pkvo_fib_record_bytes(dim, k, n_codewords, norm_format)


def turbo_record_bytes(dim, bits, mode, projections, radii_codec) -> int:
    return lib().pkvo_turbo_record_bytes(dim, bits, mode, projections, radii_codec)


def polar_lut(polar_bits):
    n = 1 << polar_bits
    c = np.empty(n, np.float32)
    s = np.empty(n, np.float32)
    lib().pkvo_polar_lut(polar_bits, _p(c, C.c_float), _p(s, C.c_float))
    return c, s


def fib_encode(x, rot, codebook, *, k=4, norm_format=0, argmin_order=0, numerics=0, nthreads=1):
    """-> (status, payload bytes array [n, rec], vec_code, vec_index)."""
    x = _f32(x)
    n, d = x.shape
    rot = np.ascontiguousarray(rot, np.float64)
    cb = _f32(codebook)
    rec = fib_record_bytes(d, k, cb.shape[0], norm_format)
    out = np.zeros((n, rec), np.uint8)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_fib_encode_batch(_p(x, C.c_float), C.c_int64(n), d, k, cb.shape[0], norm_format,
                                     argmin_order, numerics, _p(rot, C.c_double), _p(cb, C.c_float),
                                     _p(out, C.c_uint8), nthreads, C.byref(code), C.byref(idx))
    return st, out, code.value, idx.value


def fib_encode_hadamard(x, rotation_seed, codebook, *, k=4, norm_format=0, argmin_order=0, nthreads=1):
    """encode_batch of the reference's `gpu` build for a large batch (fib-quant/src/codec.rs:612-656): the
    f32 Walsh-Hadamard rotation of gpu-backend/src/fallback.rs:12-88.  -> (status, payload [n, rec], code, index)."""
    x = _f32(x)
    n, d = x.shape
    cb = _f32(codebook)
    rec = fib_record_bytes(d, k, cb.shape[0], norm_format)
    out = np.zeros((n, rec), np.uint8)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_fib_encode_batch_hadamard(_p(x, C.c_float), C.c_int64(n), d, k, cb.shape[0], norm_format,
                                              argmin_order, C.c_uint64(rotation_seed), _p(cb, C.c_float),
                                              _p(out, C.c_uint8), nthreads, C.byref(code), C.byref(idx))
    return st, out, code.value, idx.value


def hadamard_batch(data, seed):
    """gpu_backend::hadamard_batch_cpu (fallback.rs:12-62) on a copy of data [n, dim] -> [n, dim] f32."""
    out = _f32(data).copy()
    n, d = out.shape
    st = lib().pkvo_hadamard_batch(_p(out, C.c_float), C.c_int64(n), d, C.c_uint64(seed))
    if st:
        raise ValueError(f"pkvo_hadamard_batch: status {st}")
    return out


def codebook_lookup(x, codebook):
    """gpu_backend::codebook_lookup_cpu (fallback.rs:254-305) -> u32 indices [n, dim / k]."""
    x = _f32(x)
    cb = _f32(codebook)
    n, d = x.shape
    k = cb.shape[1]
    out = np.zeros((n, d // k), np.uint32)
    st = lib().pkvo_codebook_lookup(_p(x, C.c_float), _p(cb, C.c_float), C.c_int64(n), d, k, cb.shape[0],
                                    _p(out, C.c_uint32))
    if st:
        raise ValueError(f"pkvo_codebook_lookup: status {st}")
    return out


def hadamard_signs(padded_dim, seed):
    out = np.zeros(padded_dim, np.float32)
    lib().pkvo_hadamard_signs(padded_dim, C.c_uint64(seed), _p(out, C.c_float))
    return out


def fib_decode(payload, dim, rot, codebook, *, k=4, norm_format=0, nthreads=1):
    """-> (status, out [n, dim] f32, vec_code, vec_index)."""
    cb = _f32(codebook)
    rec = fib_record_bytes(dim, k, cb.shape[0], norm_format)
    payload = np.ascontiguousarray(payload, np.uint8).reshape(-1, rec)
    n = payload.shape[0]
    rot = np.ascontiguousarray(rot, np.float64)
    out = np.zeros((n, dim), np.float32)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_fib_decode_batch(_p(payload, C.c_uint8), C.c_int64(n), dim, k, cb.shape[0],
                                     norm_format, _p(rot, C.c_double), _p(cb, C.c_float),
                                     _p(out, C.c_float), C.c_int64(dim), nthreads, C.byref(code),
                                     C.byref(idx))
    return st, out, code.value, idx.value


def fib_decode_exact(payload, dim, rot, codebook, *, k=4, norm_format=0):
    """FibQuantizer::decode (binary64 inverse rotation) per record -> (status, out [n, dim] f32, code, index)."""
    cb = _f32(codebook)
    rec = fib_record_bytes(dim, k, cb.shape[0], norm_format)
    payload = np.ascontiguousarray(payload, np.uint8).reshape(-1, rec)
    n = payload.shape[0]
    rot = np.ascontiguousarray(rot, np.float64)
    out = np.zeros((n, dim), np.float32)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_fib_decode_exact_batch(_p(payload, C.c_uint8), C.c_int64(n), dim, k, cb.shape[0], norm_format,
                                           _p(rot, C.c_double), _p(cb, C.c_float), _p(out, C.c_float),
                                           C.byref(code), C.byref(idx))
    return st, out, code.value, idx.value


def turbo_encode(x, signs, qjl, *, bits=4, mode=1, radii_codec=0, libm_mode=LIBM_PORTABLE,
                 nthreads=1):
    x = _f32(x)
    n, d = x.shape
    signs = _f32(signs)
    m = 0 if qjl is None else qjl.shape[0]
    q = _f32(qjl) if qjl is not None else np.zeros(1, np.float32)
    pb = bits - 1 if mode == 1 else bits
    cl, sl = polar_lut(pb)
    rec = turbo_record_bytes(d, bits, mode, m, radii_codec)
    out = np.zeros((n, rec), np.uint8)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_turbo_encode_batch(_p(x, C.c_float), C.c_int64(n), d, bits, mode, m, radii_codec,
                                       libm_mode, _p(signs, C.c_float), _p(q, C.c_float),
                                       _p(cl, C.c_float), _p(sl, C.c_float), _p(out, C.c_uint8),
                                       nthreads, C.byref(code), C.byref(idx))
    return st, out, code.value, idx.value


def turbo_decode(payload, dim, signs, *, bits=4, mode=1, projections=32, radii_codec=0,
                 libm_mode=LIBM_PORTABLE, nthreads=1):
    rec = turbo_record_bytes(dim, bits, mode, projections, radii_codec)
    payload = np.ascontiguousarray(payload, np.uint8).reshape(-1, rec)
    n = payload.shape[0]
    signs = _f32(signs)
    pb = bits - 1 if mode == 1 else bits
    cl, sl = polar_lut(pb)
    out = np.zeros((n, dim), np.float32)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_turbo_decode_batch(_p(payload, C.c_uint8), C.c_int64(n), dim, bits, mode,
                                       projections, radii_codec, libm_mode, _p(signs, C.c_float),
                                       _p(cl, C.c_float), _p(sl, C.c_float), _p(out, C.c_float),
                                       C.c_int64(dim), nthreads, C.byref(code), C.byref(idx))
    return st, out, code.value, idx.value


def turbo_prepare_query(query, signs, qjl=None):
    """(rotated, projected) as TurboQuantizer::prepare_query returns them (turbo.rs:322-337)."""
    q, signs = _f32(query), _f32(signs)
    dim = q.size
    rotated = np.zeros(dim, np.float32)
    m = 0 if qjl is None else np.asarray(qjl).shape[0]
    projected = np.zeros(max(m, 1), np.float32)
    g = None if qjl is None else _f32(qjl)
    st = lib().pkvo_turbo_prepare_query(_p(q, C.c_float), dim, m, _p(signs, C.c_float),
                                        None if g is None else _p(g, C.c_float), _p(rotated, C.c_float),
                                        _p(projected, C.c_float))
    return st, rotated, projected[:m]


def turbo_score(payload, dim, rotated, projected, *, bits=4, mode=1, projections=32, radii_codec=0,
                libm_mode=LIBM_PORTABLE):
    """TurboQuantizer::score_batch_prepared over wire records (turbo.rs:340-381)."""
    rec = turbo_record_bytes(dim, bits, mode, projections, radii_codec)
    payload = np.ascontiguousarray(payload, np.uint8).reshape(-1, rec)
    n = payload.shape[0]
    pb = bits - 1 if mode == 1 else bits
    cl, sl = polar_lut(pb)
    rotated = _f32(rotated)
    projected = _f32(projected) if mode == 1 else np.zeros(1, np.float32)
    scores = np.zeros(n, np.float32)
    code, idx = C.c_int32(0), C.c_int64(-1)
    st = lib().pkvo_turbo_score_batch(_p(payload, C.c_uint8), C.c_int64(n), dim, bits, mode, projections,
                                      radii_codec, libm_mode, _p(cl, C.c_float), _p(sl, C.c_float),
                                      _p(rotated, C.c_float), _p(projected, C.c_float), _p(scores, C.c_float),
                                      C.byref(code), C.byref(idx))
    return st, scores, code.value, idx.value


def fb2_header(dim, n_vectors, k=4, n_codewords=32, norm_format=0) -> bytes:
    buf = (C.c_uint8 * 19)()
    lib().pkvo_fb2_header_write(dim, k, n_codewords, norm_format, C.c_uint32(n_vectors), buf)
    return bytes(buf)


def fb2_parse(data: bytes, dim, k=4, n_codewords=32, norm_format=0):
    n = C.c_uint32(0)
    arr = np.frombuffer(data, np.uint8)
    st = lib().pkvo_fb2_header_parse(dim, k, n_codewords, norm_format, _p(arr, C.c_uint8),
                                     C.c_int64(len(data)), C.byref(n))
    return st, n.value


def tqb1_header(dim, bits, mode, projections, radii_codec, seed, n_vectors) -> bytes:
    buf = (C.c_uint8 * 38)()
    lib().pkvo_tqb1_header_write(dim, bits, mode, projections, radii_codec, C.c_uint64(seed),
                                 C.c_uint32(n_vectors), buf)
    return bytes(buf)


def tqb1_parse(data: bytes, dim, bits, mode, projections, seed):
    n, codec = C.c_uint32(0), C.c_int32(0)
    arr = np.frombuffer(data, np.uint8)
    st = lib().pkvo_tqb1_header_parse(dim, bits, mode, projections, C.c_uint64(seed),
                                      _p(arr, C.c_uint8), C.c_int64(len(data)), C.byref(n),
                                      C.byref(codec))
    return st, n.value, codec.value
