"""ctypes binding of libprovekv_b200.so (the C ABI in include/provekv_b200.h).

There is no CPU fallback: if the shared library is missing the import of the
symbols fails with an explicit error, and every compute call fails with
PKV_ERR_CUDA when no CUDA device is usable.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_PKG, "libprovekv_b200.so")

# status codes (include/provekv_b200.h)
OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_CUDA = 2
ERR_UNSUPPORTED = 3
ERR_EMPTY_BATCH = 4
ERR_CORRUPT_HEADER = 5
ERR_BUFFER_TOO_SMALL = 6
ERR_STATIC_SCRATCH_TOO_SMALL = 7
VEC_NONFINITE_INPUT = 16
VEC_ZERO_NORM = 17
VEC_BAD_RADIUS = 18
VEC_BAD_RADIUS_RANGE = 19
VEC_PADDING_BITS = 20
VEC_INDEX_RANGE = 21
VEC_BAD_NORM = 22
VEC_NONFINITE_OUTPUT = 23
VEC_NONFINITE_RESIDUAL = 24
VEC_NORM_RANGE = 25
VEC_DEVICE_WAIT = 26
VEC_MISALIGNED_DST = 27

NORM_FP16, NORM_F32 = 0, 1
ARGMIN_PAIRWISE, ARGMIN_SEQUENTIAL = 0, 1
FIB_NUMERICS_AUTO, FIB_NUMERICS_BATCH, FIB_NUMERICS_SINGLE = 0, 1, 2
TURBO_POLAR_ONLY, TURBO_POLAR_WITH_QJL = 0, 1
RADII_F32, RADII_BLOCK_LOG_U8 = 0, 1
LIBM_PORTABLE, LIBM_PLATFORM = 0, 1
DST_F32, DST_F16, DST_BF16 = 0, 1, 2  # PKV_DST_*: element type of the patched cache
FB2_HEADER_BYTES, TQB1_HEADER_BYTES = 19, 38


class FibConfigC(C.Structure):
    _fields_ = [("dim", C.c_int32), ("block_dim", C.c_int32), ("codebook_size", C.c_int32),
                ("norm_format", C.c_int32), ("argmin_order", C.c_int32), ("numerics", C.c_int32)]


class TurboConfigC(C.Structure):
    _fields_ = [("dim", C.c_int32), ("bits", C.c_int32), ("mode", C.c_int32),
                ("projections", C.c_int32), ("radii_codec", C.c_int32), ("libm", C.c_int32),
                ("seed", C.c_uint64)]


class Layout(C.Structure):
    """pkv_layout: where the vectors of a launch live in an f32 tensor (elements)."""
    _fields_ = [("base", C.c_int64), ("batch_stride", C.c_int64 * 3), ("token_stride", C.c_int64),
                ("head_stride", C.c_int64), ("replica_stride", C.c_int64),
                ("n_batches", C.c_int32 * 3), ("n_tokens", C.c_int32), ("n_heads", C.c_int32),
                ("n_replicas", C.c_int32)]

    @classmethod
    def make(cls, *, n_tokens, n_heads, token_stride, head_stride, base=0, n_batches=(1, 1, 1),
             batch_stride=(0, 0, 0), n_replicas=1, replica_stride=0) -> "Layout":
        L = cls()
        L.base = base
        L.batch_stride = (C.c_int64 * 3)(*batch_stride)
        L.token_stride = token_stride
        L.head_stride = head_stride
        L.replica_stride = replica_stride
        L.n_batches = (C.c_int32 * 3)(*n_batches)
        L.n_tokens = n_tokens
        L.n_heads = n_heads
        L.n_replicas = n_replicas
        return L

    @property
    def vectors_per_batch(self) -> int:
        return self.n_tokens * self.n_heads

    @property
    def batch_count(self) -> int:
        return self.n_batches[0] * self.n_batches[1] * self.n_batches[2]


class PkvError(RuntimeError):
    """A non-zero status from the library; ``vector_index`` is set for per-vector codes."""

    def __init__(self, status: int, message: str, vector_index: int = -1):
        super().__init__(f"{message} (status {status}" +
                         (f", vector {vector_index})" if vector_index >= 0 else ")"))
        self.status = status
        self.vector_index = vector_index


def build(verbose: bool = False) -> str:
    """Compile the CUDA library in-tree for sm_100a (provekv_b200/csrc/Makefile)."""
    r = subprocess.run(["make", "-C", os.path.join(_PKG, "csrc")], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode != 0:
        raise RuntimeError("building libprovekv_b200.so failed")
    return SO_PATH


_lib = None

_V = C.c_void_p
_SIGS = {
    "pkv_status_string": (C.c_char_p, [C.c_int]),
    "pkv_version": (C.c_int, []),
    "pkv_last_cuda_error": (C.c_char_p, []),
    "pkv_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "pkv_set_device": (C.c_int, [C.c_int]),
    "pkv_host_alloc": (C.c_int, [C.POINTER(_V), C.c_int64]),
    "pkv_host_free": (C.c_int, [_V]),
    "pkv_dev_alloc": (C.c_int, [C.POINTER(_V), C.c_int64]),
    "pkv_dev_free": (C.c_int, [_V]),
    "pkv_memcpy_h2d": (C.c_int, [_V, _V, C.c_int64, _V]),
    "pkv_memcpy_d2h": (C.c_int, [_V, _V, C.c_int64, _V]),
    "pkv_stream_synchronize": (C.c_int, [_V]),
    "pkv_payload_upload": (C.c_int, [_V, C.c_int64, C.c_int32, C.c_int64, C.c_int64, _V, C.c_int64, _V]),
    "pkv_payload_download": (C.c_int, [_V, C.c_int64, C.c_int64, C.c_int64, _V, C.c_int64, C.c_int32, _V]),
    "pkv_test_capture_rotated": (C.c_int, [_V]),
    "pkv_stats_read": (C.c_int, [C.POINTER(C.c_uint64)]),
    "pkv_stats_reset": (C.c_int, []),
    "pkv_error_word_reset": (C.c_int, [_V, _V]),
    "pkv_error_word_read": (C.c_int, [_V, _V, C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_hadamard_batch_dev": (C.c_int, [_V, C.c_int64, C.c_int32, C.c_uint64, _V]),
    "pkv_codebook_lookup_batch_dev": (C.c_int, [_V, _V, C.c_int64, C.c_int32, C.c_int32, C.c_int32, _V, _V]),
    "pkv_fib_profile_create": (C.c_int, [C.POINTER(FibConfigC), _V, _V, C.POINTER(_V)]),
    "pkv_fib_profile_create_hadamard": (C.c_int, [C.POINTER(FibConfigC), C.c_uint64, _V, _V, C.POINTER(_V)]),
    "pkv_fib_profile_destroy": (C.c_int, [_V]),
    "pkv_fib_record_bytes": (C.c_int32, [_V]),
    "pkv_fib_encode_dev": (C.c_int, [_V, _V, C.POINTER(Layout), _V, C.c_int64, _V, _V]),
    "pkv_fib_decode_patch_dev": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, _V, _V]),
    "pkv_fib_decode_exact_dev": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, _V, _V]),
    "pkv_fib_decode_exact": (C.c_int, [_V, _V, C.c_int64, _V, C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_fib_decode_patch_dev_as": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, C.c_int32, _V, _V]),
    "pkv_turbo_decode_patch_dev_as": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, C.c_int32, _V, _V]),
    "pkv_fib_decode_patch_dev_multi": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, _V, C.c_int32, _V, _V]),
    "pkv_turbo_decode_patch_dev_multi": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, _V, C.c_int32, _V, _V]),
    "pkv_turbo_score_dev": (C.c_int, [_V, _V, C.c_int64, C.c_int64, C.c_int64, _V, _V, _V, _V, _V]),
    "pkv_turbo_score_queries_dev": (C.c_int, [_V, _V, C.c_int64, C.c_int64, C.c_int64, _V, _V, C.c_int64, _V, _V, _V]),
    "pkv_turbo_prepare_queries_dev": (C.c_int, [_V, _V, C.c_int64, _V, _V, _V, _V]),
    "pkv_fib_encode_dev_static": (C.c_int, [_V, _V, C.POINTER(Layout), _V, C.c_int64, _V, _V]),
    "pkv_fib_encode_batch_compact": (C.c_int, [_V, _V, C.c_int64, _V, C.c_int64, C.POINTER(C.c_int64),
                                               C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_fib_decode_batch_compact": (C.c_int, [_V, _V, C.c_int64, _V, C.c_int64, C.POINTER(C.c_int64),
                                               C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_fb2_header_write": (C.c_int, [_V, C.c_uint32, _V]),
    "pkv_fb2_header_parse": (C.c_int, [_V, _V, C.c_int64, C.POINTER(C.c_uint32)]),
    "pkv_turbo_profile_create": (C.c_int, [C.POINTER(TurboConfigC), _V, _V, _V, _V, C.POINTER(_V)]),
    "pkv_turbo_profile_destroy": (C.c_int, [_V]),
    "pkv_turbo_record_bytes": (C.c_int32, [_V]),
    "pkv_turbo_encode_dev": (C.c_int, [_V, _V, C.POINTER(Layout), _V, C.c_int64, _V, _V]),
    "pkv_turbo_decode_patch_dev": (C.c_int, [_V, _V, C.c_int64, C.POINTER(Layout), _V, _V, _V]),
    "pkv_turbo_encode_batch_compact": (C.c_int, [_V, _V, C.c_int64, _V, C.c_int64, C.POINTER(C.c_int64),
                                                 C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_turbo_decode_batch_compact": (C.c_int, [_V, _V, C.c_int64, _V, C.c_int64, C.POINTER(C.c_int64),
                                                 C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_tqb1_header_write": (C.c_int, [_V, C.c_uint32, _V]),
    "pkv_tqb1_header_parse": (C.c_int, [_V, _V, C.c_int64, C.POINTER(C.c_uint32)]),
    "pkv_host_libm_exceptions": (C.c_int, [C.c_int32, _V, C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int32)]),
    "pkv_launch_count": (C.c_int64, []),
    "pkv_test_skip_tensor_issue": (C.c_int, [C.c_int]),
    "pkv_test_turbo_encode_legacy": (C.c_int, [C.c_int]),
    "pkv_fib_encode_batches_compact": (C.c_int, [_V, _V, C.c_int64, C.c_int64, _V, C.c_int64,
                                                 C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_fib_decode_batches_compact": (C.c_int, [_V, _V, C.c_int64, C.c_int64, _V, C.c_int64,
                                                 C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_turbo_encode_batches_compact": (C.c_int, [_V, _V, C.c_int64, C.c_int64, _V, C.c_int64,
                                                   C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "pkv_turbo_decode_batches_compact": (C.c_int, [_V, _V, C.c_int64, C.c_int64, _V, C.c_int64,
                                                   C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
}

EXPORTED_SYMBOLS = tuple(_SIGS)


def lib() -> C.CDLL:
    """Load the CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(
                f"{SO_PATH} is missing: build it with `make -C provekv_b200/csrc` "
                "(there is no CPU implementation to fall back to)")
        L = C.CDLL(SO_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def status_string(status: int) -> str:
    text = lib().pkv_status_string(status).decode()
    if status == ERR_CUDA:
        detail = lib().pkv_last_cuda_error().decode()
        if detail:
            text += f": {detail}"
    return text


def check(status: int, vector_index: int = -1) -> None:
    if status != OK:
        raise PkvError(status, status_string(status), vector_index)
