"""include/pkv_portable_math.h: accuracy, special cases, and how often it differs
from the host libm (the quantity that decides "bit-exact with the reference on this
machine" for the angle buckets and the BlockLogU8 radii)."""
import ctypes as C
import math

import mpmath as mp
import numpy as np

PORTABLE, PLATFORM = 1, 0


def _f32(x):
    return float(np.float32(x))


def test_atan2_special_cases_follow_c_annex_f(oracle_mod):
    f = oracle_mod.lib().pkvo_atan2f
    pi = _f32(math.pi)
    assert f(0.0, 1.0, PORTABLE) == 0.0 and math.copysign(1, f(0.0, 1.0, PORTABLE)) == 1
    assert math.copysign(1, f(-0.0, 1.0, PORTABLE)) == -1
    assert f(0.0, -1.0, PORTABLE) == pi and f(-0.0, -1.0, PORTABLE) == -pi
    assert f(0.0, 0.0, PORTABLE) == 0.0 and f(0.0, -0.0, PORTABLE) == pi
    assert f(-0.0, -0.0, PORTABLE) == -pi
    assert f(1.0, 0.0, PORTABLE) == _f32(math.pi / 2) and f(-1.0, -0.0, PORTABLE) == -_f32(math.pi / 2)
    for y, x in [(0.0, 1.0), (-0.0, 1.0), (0.0, -1.0), (-0.0, -1.0), (0.0, 0.0), (0.0, -0.0),
                 (-0.0, -0.0), (-0.0, 0.0), (1.0, 0.0), (-1.0, -0.0), (1.0, 1.0), (-3.0, -3.0)]:
        a, b = f(y, x, PORTABLE), f(y, x, PLATFORM)
        assert a == b and math.copysign(1, a) == math.copysign(1, b), (y, x)


def test_portable_functions_are_correctly_rounded_on_samples(oracle_mod):
    L = oracle_mod.lib()
    rng = np.random.default_rng(0)
    mp.mp.prec = 120
    ys = rng.standard_normal(3000).astype(np.float32) * np.float32(3)
    xs = rng.standard_normal(3000).astype(np.float32) * np.float32(3)
    for y, x in zip(ys, xs):
        want = _f32(mp.atan2(mp.mpf(float(y)), mp.mpf(float(x))))
        assert L.pkvo_atan2f(float(y), float(x), PORTABLE) == want
    rs = np.exp(rng.uniform(-80, 80, 3000)).astype(np.float32)
    for r in rs:
        assert L.pkvo_logf(float(r), PORTABLE) == _f32(mp.log(mp.mpf(float(r))))
    ts = rng.uniform(-100, 88, 3000).astype(np.float32)
    for t in ts:
        assert L.pkvo_expf(float(t), PORTABLE) == _f32(mp.exp(mp.mpf(float(t))))
    assert L.pkvo_expf(100.0, PORTABLE) == float("inf")
    assert L.pkvo_expf(-200.0, PORTABLE) == 0.0
    assert L.pkvo_logf(_f32(1.17549435e-38), PORTABLE) == _f32(mp.log(mp.mpf(_f32(1.17549435e-38))))


def test_bucket_disagreement_with_host_libm_is_rare(oracle_mod):
    """Angle bucket from the portable atan2f vs from the host libm's atan2f: the bucket can only
    differ when the two results straddle a bucket threshold, i.e. almost never."""
    L = oracle_mod.lib()
    rng = np.random.default_rng(1)
    n = 200_000
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    diff_theta = diff_bucket = 0
    for y, x in zip(b.tolist(), a.tolist()):
        t0, t1 = L.pkvo_atan2f(y, x, PORTABLE), L.pkvo_atan2f(y, x, PLATFORM)
        if t0 != t1:
            diff_theta += 1
            for levels in (8, 16):
                if L.pkvo_angle_bucket(t0, levels) != L.pkvo_angle_bucket(t1, levels):
                    diff_bucket += 1
    assert diff_theta / n < 0.3       # the libm is within 1 ulp but not correctly rounded
    assert diff_bucket <= 2           # expected ~1e-7 per pair


def test_bucket_thresholds_monotone(oracle_mod):
    """The bucket is a monotone step function of theta with exactly `levels` steps on [-pi, pi]."""
    L = oracle_mod.lib()
    for levels in (2, 8, 16, 128):
        thetas = np.linspace(-math.pi, math.pi, 20001).astype(np.float32)
        idx = np.array([L.pkvo_angle_bucket(float(t), levels) for t in thetas])
        raw = idx.copy()
        raw[-1] = levels if idx[-1] == 0 else idx[-1]  # theta = +pi wraps to bucket 0
        assert np.all(np.diff(raw.astype(np.int64)) >= 0)
        assert idx.max() == levels - 1 and idx.min() == 0
    assert L.pkvo_angle_bucket(_f32(math.pi), 8) == 0   # normalized == 1.0 -> levels % levels
    assert L.pkvo_angle_bucket(0.0, 8) == 4


def test_host_libm_exception_lists_are_exact(oracle_mod):
    """pkv_host_libm_exceptions: the library's scan of every binary32 argument for the inputs on which
    the host logf / expf and the portable functions differ.  Checked against the oracle's two libm
    modes: every listed argument differs by exactly one unit, and a random sample of unlisted
    arguments does not differ at all."""
    from provekv_b200 import _lib as L
    lib, O = L.lib(), oracle_mod.lib()
    rng = np.random.default_rng(1)
    for fn, name, lo, hi in ((0, "pkvo_logf", 0x00800000, 0x7f7fffff), (1, "pkvo_expf", 0, 0x42b20000)):
        n, ok = C.c_int64(0), C.c_int32(0)
        assert lib.pkv_host_libm_exceptions(fn, None, 0, C.byref(n), C.byref(ok)) == L.OK
        assert ok.value == 1 and 1000 < n.value < 5_000_000
        keys = np.zeros(n.value, np.uint32)
        assert lib.pkv_host_libm_exceptions(fn, keys.ctypes.data_as(C.c_void_p), n.value, C.byref(n), None) == L.OK
        assert np.all(np.diff(keys.astype(np.int64)) > 0)
        f = getattr(O, name)
        for k in keys[rng.integers(0, keys.size, 2000)]:
            x = float(np.array([k], np.uint32).view(np.float32)[0])
            a = np.float32(f(x, PORTABLE)).view(np.uint32).astype(np.int64)
            b = np.float32(f(x, PLATFORM)).view(np.uint32).astype(np.int64)
            assert abs(int(a) - int(b)) == 1, hex(int(k))
        listed = set(keys.tolist())
        sample = rng.integers(lo, hi, 4000, dtype=np.uint32)
        if fn == 1:
            sample = sample | (rng.integers(0, 2, 4000, dtype=np.uint32) << np.uint32(31))
        for k in sample:
            if int(k) in listed:
                continue
            x = float(np.array([k], np.uint32).view(np.float32)[0])
            assert np.float32(f(x, PORTABLE)).view(np.uint32) == np.float32(f(x, PLATFORM)).view(np.uint32), hex(int(k))
