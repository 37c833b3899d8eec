"""The C-ABI library loads without a GPU and exports every symbol the header declares.
No compute call is made here (there is no CPU implementation behind the ABI)."""
import ctypes as C
import os
import re
import subprocess

import provekv_b200 as pk
from provekv_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "provekv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pkv_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_loads():
    L.build()
    assert os.path.exists(L.SO_PATH)
    assert L.lib().pkv_version() >= 100


def test_every_declared_symbol_is_exported_and_bound():
    declared = _declared_symbols()
    assert len(declared) >= 30
    lib = C.CDLL(L.SO_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert sorted(L.EXPORTED_SYMBOLS) == declared
    nm = subprocess.run(["nm", "-D", "--defined-only", L.SO_PATH], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (pkv_[a-z0-9_]+)", nm))
    assert set(declared) <= exported


def test_status_strings_and_argument_checks_need_no_gpu():
    lib = L.lib()
    assert L.status_string(L.OK) == "ok"
    for code in list(range(0, 8)) + list(range(16, 26)):
        assert L.status_string(code) != "unknown status"
    assert L.status_string(99) == "unknown status"
    n = C.c_uint32(0)
    assert lib.pkv_fb2_header_parse(None, None, 0, C.byref(n)) == L.ERR_INVALID_ARGUMENT
    assert lib.pkv_tqb1_header_parse(None, None, 0, C.byref(n)) == L.ERR_INVALID_ARGUMENT
    assert lib.pkv_fib_record_bytes(None) == 0 and lib.pkv_turbo_record_bytes(None) == 0
    h = C.c_void_p()
    assert lib.pkv_fib_profile_create(None, None, None, C.byref(h)) == L.ERR_INVALID_ARGUMENT
    cfg = L.FibConfigC(48, 4, 32, 0, 0, 0)  # a dim the kernels are not built for
    import numpy as np
    rot, cb = np.eye(48), np.zeros((32, 4), np.float32)
    assert lib.pkv_fib_profile_create(C.byref(cfg), rot.ctypes.data_as(C.c_void_p),
                                      cb.ctypes.data_as(C.c_void_p), C.byref(h)) == L.ERR_UNSUPPORTED
    assert lib.pkv_launch_count() == 0


def test_python_mirror_of_the_reference_interface():
    # names and argument checks of proveKV/src/codec.rs
    import pytest
    with pytest.raises(pk.InvalidPolicy):
        pk.FibQuantAdapter(0, 4, 32, 2048, 4, 8)
    with pytest.raises(pk.InvalidPolicy):
        pk.FibQuantAdapter(66, 4, 32, 2048, 4, 8)
    with pytest.raises(pk.InvalidPolicy):
        pk.TurboQuantAdapter(63, 4, 32)
    with pytest.raises(pk.InvalidPolicy):
        pk.create_codec("nope", 64)
    with pytest.raises(pk.InvalidPolicy):
        pk.create_codec(pk.CODEC_FIB_K4_N32, 64)
    fib = pk.create_codec(pk.CODEC_FIB_K4_N32_BATCHED, 64, fib_config=pk.FibConfig())
    assert isinstance(fib, pk.FibQuantAdapter) and fib.codec_id() == "fib_k4_n32" and fib.dim() == 64
    tq = pk.create_codec(pk.CODEC_TURBO_8BIT, 64, turbo_config=pk.TurboConfig())
    assert isinstance(tq, pk.TurboQuantAdapter) and tq.bits == 4 and tq.projections == 32
    assert pk.turbo_batched_codec_id(4, True) == "turbo_4bit_batched_lossy"
    assert pk.turbo_batched_codec_id(8, False) == "turbo_8bit_batched"
