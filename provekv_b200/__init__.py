"""provekv_b200: proveKV's KV-cache codec hot path (fib-quant FB2, turbo-quant TQB1,
fused decode-and-patch) as hand-written CUDA kernels for B200 (sm_100a) behind a C ABI.

The CUDA library is the only implementation: importing the package is cheap and
works without a GPU, but every codec call needs ``libprovekv_b200.so`` (built
in-tree by ``provekv_b200._lib.build()`` / ``make -C provekv_b200/csrc``) and a CUDA device.
"""
from . import _lib, kv_pages, manifest, patch, records, rust_streams, tables
from ._lib import Layout, PkvError
from .codec import (CODEC_FIB_K4_N32, CODEC_FIB_K4_N32_BATCHED, CODEC_TURBO_8BIT,
                    CODEC_TURBO_8BIT_BATCHED, CompressionFailed, DecompressionFailed, FibConfig,
                    FibQuantAdapter, InvalidPolicy, KVecCodec, ProveKvError, TurboConfig,
                    TurboQuantAdapter, create_codec, turbo_batched_codec_id)
from .profiles import (FibProfile, TurboProfile, decode_batches_compact, encode_batches_compact,
                       read_error_word)

__all__ = [n for n in dir() if not n.startswith("_")]
