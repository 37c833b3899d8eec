"""Failure paths and guard rails of the CUDA library, exercised without faulting the GPU:
a bounded wait that runs out, a profile used from the wrong device, a rotation table that is
not orthonormal, residuals too small for binary32 norms, and the error word's order when one
launch covers several batches.
"""
import ctypes as C

import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import tables

from kvgen import synthetic_kv

pytestmark = pytest.mark.gpu

SEED = 42


def _flat_layout(n_batches, vpb, dim):
    return L.Layout.make(n_batches=(n_batches, 1, 1), batch_stride=(vpb * dim, 0, 0), n_tokens=vpb,
                         n_heads=1, token_stride=dim, head_stride=dim)


@pytest.mark.parametrize("codec,dim", [("turbo", 64), ("fib", 64), ("fib", 128)])
def test_bounded_wait_runs_out_and_the_context_stays_usable(oracle_mod, codec, dim):
    """With the tensor-core products withheld (test hook) the completion barrier never flips: the
    kernels poll it a few hundred times, report PKV_VEC_DEVICE_WAIT, give their tensor memory back
    and return.  Afterwards the same profile encodes normally and matches the oracle."""
    n = 5000
    x = synthetic_kv(n, dim, seed=3)
    if codec == "turbo":
        signs, qjl = tables.rademacher_signs(dim, SEED), tables.qjl_matrix(dim, 32, SEED)
        prof = pk.TurboProfile(dim, 4, signs, qjl, seed=SEED)
    else:
        rot, cb = tables.haar_rotation(dim, SEED), tables.fib_codebook(dim, seed=SEED)
        prof = pk.FibProfile(dim, rot, cb)
    lib = L.lib()
    assert lib.pkv_test_skip_tensor_issue(1) == L.OK
    try:
        with pytest.raises(L.PkvError) as ei:
            prof.encode_batch_compact(x)
        assert ei.value.status == L.VEC_DEVICE_WAIT
    finally:
        lib.pkv_test_skip_tensor_issue(0)
    got = prof.encode_batch_compact(x)
    if codec == "turbo":
        st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=4, mode=1, radii_codec=0,
                                                   libm_mode=oracle_mod.LIBM_PORTABLE)
        assert st == 0 and got[L.TQB1_HEADER_BYTES:] == payload.tobytes()
    else:
        st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb)
        assert st == 0 and got[L.FB2_HEADER_BYTES:] == payload.tobytes()


def test_profile_is_bound_to_its_device():
    """A profile's tables live on the device it was created on; calls made with another device
    current are refused before anything is launched or copied."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = L.lib()
    dim, n = 64, 256
    L.check(lib.pkv_set_device(0))
    fib = pk.FibProfile(dim, tables.haar_rotation(dim, 1), tables.fib_codebook(dim, seed=1))
    tq = pk.TurboProfile(dim, 4, tables.rademacher_signs(dim, 1), tables.qjl_matrix(dim, 32, 1), seed=1)
    x = synthetic_kv(n, dim, seed=1)
    fib_wire, tq_wire = fib.encode_batch_compact(x), tq.encode_batch_compact(x)
    L.check(lib.pkv_set_device(1))
    try:
        launches = lib.pkv_launch_count()
        with torch.cuda.device(1):
            xd = torch.from_numpy(x).cuda()
            out = torch.zeros(n * 256, dtype=torch.uint8, device="cuda")
            err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
            lay = _flat_layout(1, n, dim)
            for prof in (fib, tq):
                with pytest.raises(L.PkvError) as ei:
                    prof.encode_dev(xd.data_ptr(), lay, out.data_ptr(), n * 256, err.data_ptr())
                assert ei.value.status == L.ERR_INVALID_ARGUMENT
                with pytest.raises(L.PkvError) as ei:
                    prof.decode_patch_dev(out.data_ptr(), n * 256, lay, xd.data_ptr(), err.data_ptr())
                assert ei.value.status == L.ERR_INVALID_ARGUMENT
                with pytest.raises(L.PkvError) as ei:
                    prof.encode_batch_compact(x)
                assert ei.value.status == L.ERR_INVALID_ARGUMENT
            st = lib.pkv_fib_encode_dev_static(fib.handle, xd.data_ptr(), C.byref(lay), out.data_ptr(),
                                               n * 256, err.data_ptr(), None)
            assert st == L.ERR_INVALID_ARGUMENT
            with pytest.raises(L.PkvError):
                fib.decode_batch_compact(fib_wire)
            with pytest.raises(L.PkvError):
                tq.decode_batch_compact(tq_wire)
            rq = torch.zeros(2 * dim, dtype=torch.float32, device="cuda")
            pq = torch.zeros(2 * 32, dtype=torch.float32, device="cuda")
            sc = torch.zeros(2 * n, dtype=torch.float32, device="cuda")
            with pytest.raises(L.PkvError) as ei:
                tq.prepare_queries_dev(xd.data_ptr(), 2, rq.data_ptr(), pq.data_ptr(), err.data_ptr())
            assert ei.value.status == L.ERR_INVALID_ARGUMENT
            with pytest.raises(L.PkvError) as ei:
                tq.score_queries_dev(out.data_ptr(), n * 256, 1, n, rq.data_ptr(), pq.data_ptr(), 2, sc.data_ptr(),
                                     err.data_ptr())
            assert ei.value.status == L.ERR_INVALID_ARGUMENT
            torch.cuda.synchronize()
            assert int(err[0]) == -1
        assert lib.pkv_launch_count() == launches
    finally:
        L.check(lib.pkv_set_device(0))
    assert fib.encode_batch_compact(x) == fib_wire


@pytest.mark.parametrize("kind", ["scaled", "sheared"])
def test_fib_matrix_that_is_not_orthonormal_takes_the_exact_kernel(oracle_mod, kind):
    """The shortcut encoders' bounds assume an orthonormal rotation.  A scaled or sheared matrix is
    still a valid table for the reference's arithmetic: such a profile encodes with the exact f64
    kernel and the bytes equal the oracle's; the no-allocation entry point refuses it."""
    import torch
    dim, n = 64, 3000
    rot, cb = tables.haar_rotation(dim, 9), tables.fib_codebook(dim, seed=9)
    rot = np.array(rot, np.float64)
    if kind == "scaled":
        rot = rot * 1.37
    else:
        rot[3] += 0.25 * rot[11]
    x = synthetic_kv(n, dim, seed=77)
    prof = pk.FibProfile(dim, rot, cb)
    got = prof.encode_batch_compact(x)
    st, payload, _, _ = oracle_mod.fib_encode(x, rot, cb)
    assert st == 0 and got[L.FB2_HEADER_BYTES:] == payload.tobytes()
    dec = prof.decode_batch_compact(got)
    st, want, _, _ = oracle_mod.fib_decode(payload, dim, rot, cb)
    assert st == 0 and np.array_equal(dec.view(np.uint32), want.view(np.uint32))
    xd = torch.from_numpy(x).cuda()
    out = torch.zeros(n * 16, dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    lay = _flat_layout(1, n, dim)
    st = L.lib().pkv_fib_encode_dev_static(prof.handle, xd.data_ptr(), C.byref(lay), out.data_ptr(), n * 16,
                                           err.data_ptr(), None)
    assert st == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("scale", [1e-25, 3e-33])
def test_turbo_residuals_below_the_binary32_norm_range(oracle_mod, dim, scale):
    """Inputs so small that the residual's squared norm underflows to zero in binary32 while the
    residual itself is not zero: the tensor-core dots flush, no bound certifies anything, and every
    sign has to come from the exact sequential dot."""
    n, m = 700, 32
    signs, qjl = tables.rademacher_signs(dim, SEED), tables.qjl_matrix(dim, m, SEED)
    x = (synthetic_kv(n, dim, seed=12).astype(np.float64) * scale).astype(np.float32)
    x[17] = 0.0
    for rc in (L.RADII_F32, L.RADII_BLOCK_LOG_U8):
        prof = pk.TurboProfile(dim, 4, signs, qjl, radii_codec=rc, seed=SEED)
        got = prof.encode_batch_compact(x)
        st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=4, mode=1, radii_codec=rc,
                                                   libm_mode=oracle_mod.LIBM_PORTABLE)
        assert st == 0
        have = np.frombuffer(got, np.uint8)[L.TQB1_HEADER_BYTES:].reshape(n, -1)
        want = payload.reshape(n, -1)
        assert np.array_equal(have, want), f"{(have != want).any(axis=1).sum()} records differ"


def test_error_word_order_over_two_batches():
    """One launch over two batches: batch 0 holds a vector whose norm overflows fp16 (found by the
    encoder's second pass), batch 1 a NaN (first pass).  Encoded one batch per call, as the reference
    does, each batch reports its own error; in one launch the word orders by pass before vector, so
    the first-pass error of the later batch is the one reported."""
    import torch
    dim, vpb = 64, 500
    rot, cb = tables.haar_rotation(dim, 5), tables.fib_codebook(dim, seed=5)
    prof = pk.FibProfile(dim, rot, cb)
    x = synthetic_kv(2 * vpb, dim, seed=8).reshape(2, vpb, dim)
    x[0, 123] *= np.float32(1e5)       # norm ~ 8e5 > 65504
    x[1, 45, 7] = np.float32("nan")
    xd = torch.from_numpy(x).cuda()
    stride = (vpb * prof.record_bytes + 15) // 16 * 16
    out = torch.zeros((2, stride), dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")

    def run(first, count):
        err.fill_(-1)
        lay = _flat_layout(count, vpb, dim)
        prof.encode_dev(xd[first:].data_ptr(), lay, out.data_ptr(), stride, err.data_ptr())
        with pytest.raises(L.PkvError) as ei:
            pk.read_error_word(err.data_ptr())
        return ei.value.status, ei.value.vector_index

    assert run(0, 1) == (L.VEC_NORM_RANGE, 123)
    assert run(1, 1) == (L.VEC_NONFINITE_INPUT, 45)
    assert run(0, 2) == (L.VEC_NONFINITE_INPUT, vpb + 45)


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("bits,m", [(4, 32), (8, 32), (3, 64)])
def test_rotated_domain_sketch_equals_the_residual_sketch(oracle_mod, dim, bits, m):
    """The two routes to the QJL signs -- the sketch of q = y - p with G S H~ (default for f32 radii) and
    the sketch of the residual after the inverse transform -- give the same records, which are the
    oracle's; outlier channels and a zero vector included."""
    n = 20000
    signs, qjl = tables.rademacher_signs(dim, SEED), tables.qjl_matrix(dim, m, SEED)
    x = synthetic_kv(n, dim, seed=31)
    x[:, 3] *= np.float32(20.0)
    x[77] = 0.0
    prof = pk.TurboProfile(dim, bits, signs, qjl, seed=SEED)
    lib = L.lib()
    got = prof.encode_batch_compact(x)
    lib.pkv_test_turbo_encode_legacy(1)
    try:
        legacy = prof.encode_batch_compact(x)
    finally:
        lib.pkv_test_turbo_encode_legacy(0)
    assert got == legacy
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=bits, mode=1, radii_codec=0,
                                               libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0 and got[L.TQB1_HEADER_BYTES:] == payload.tobytes()


def test_pool_built_on_the_device_it_names():
    """build_shared_pool puts data, stream and launch on the device it is given: a profile that lives
    on that device encodes there whatever device is current, and a profile from another device is refused
    with the library's status instead of faulting."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from provekv_b200 import manifest as M
    lib = L.lib()
    d, H, Lc, T = 64, 2, 2, 19
    shape = M.KvTensorShape("gqa", Lc, 8, H, d, 8 * d)
    corpus = synthetic_kv(T * Lc * H * 2, d, seed=4).reshape(T, Lc * H * 2 * d)
    L.check(lib.pkv_set_device(1))
    try:
        with torch.cuda.device(1):
            prof1 = pk.FibProfile(d, tables.haar_rotation(d, 2), tables.fib_codebook(d, seed=2))
    finally:
        L.check(lib.pkv_set_device(0))
    prof0 = pk.FibProfile(d, tables.haar_rotation(d, 2), tables.fib_codebook(d, seed=2))
    on1 = M.build_shared_pool(prof1, corpus, shape, 7, "cb", "rot", device="cuda:1", built_at_unix=1)
    on0 = M.build_shared_pool(prof0, corpus, shape, 7, "cb", "rot", device="cuda:0", built_at_unix=1)
    assert on1["pool_id"] == on0["pool_id"] and torch.cuda.current_device() == 0
    with pytest.raises(L.PkvError) as ei:
        M.build_shared_pool(prof1, corpus, shape, 7, "cb", "rot", device="cuda:0")
    assert ei.value.status == L.ERR_INVALID_ARGUMENT


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("numerics,norm_format,hadamard", [(1, 0, False), (2, 0, False), (1, 1, False), (1, 0, True)])
def test_refused_vectors_leave_zero_records_and_the_rest_intact(oracle_mod, dim, numerics, norm_format, hadamard):
    """A per-vector status from the batched host call still delivers the whole payload: refused vectors as
    all-zero records, every other record as if the refused vectors had not been there."""
    import numpy as np
    from provekv_b200 import _lib as L
    from provekv_b200 import tables
    from provekv_b200.profiles import FibProfile, encode_batches_compact
    from kvgen import synthetic_kv
    rot, cb = tables.haar_rotation(dim, 42), tables.fib_codebook(dim, seed=42)
    prof = FibProfile(dim, rot, cb, numerics=numerics, norm_format=norm_format, hadamard_seed=7 if hadamard else None)
    nb, vpb = 3, 700
    x = synthetic_kv(nb * vpb, dim, seed=11)
    bad = {5: 0.0, 701: None, 1399: 0.0, 2099: np.nan}        # 701: finite elements, norm beyond the wire format
    clean = x.copy()
    for i, v in bad.items():
        x[i] = (np.sign(x[i]) * np.float32(3e38) if norm_format else x[i] * np.float32(3e4)) if v is None else v
        clean[i] = 0.0
        clean[i, 0] = 1.0
    H, rec = L.FB2_HEADER_BYTES, prof.record_bytes
    out = np.full((nb, H + vpb * rec), 0xAB, np.uint8)
    with pytest.raises(L.PkvError) as e:
        encode_batches_compact(prof, x.ctypes.data, nb, vpb, out.ctypes.data, out.size)
    # the reference's first loop (non-finite, zero norm) reports before the norm format is looked at
    assert e.value.status in (L.VEC_ZERO_NORM, L.VEC_NONFINITE_INPUT) and e.value.vector_index == 5
    got = out[:, H:].reshape(nb * vpb, rec)
    if hadamard:
        st, want, _, _ = oracle_mod.fib_encode_hadamard(clean, 7, cb, norm_format=norm_format, nthreads=4)
    else:
        st, want, _, _ = oracle_mod.fib_encode(clean, rot, cb, norm_format=norm_format, numerics=numerics, nthreads=4)
    assert st == 0
    keep = np.ones(nb * vpb, bool)
    keep[list(bad)] = False
    assert np.array_equal(got[keep], want[keep])
    assert not got[~keep].any()


@pytest.mark.gpu
def test_tier_counters_count_what_the_shortcuts_did_not_settle():
    """pkv_stats_read: after a reset and one encode of each codec the counters hold a small, non-zero share
    of the work (the shortcuts settle almost everything), and a reset clears them."""
    import numpy as np
    lib = L.lib()
    dim, n = 64, 40_000
    x = synthetic_kv(n, dim, seed=21)
    fib = pk.FibProfile(dim, tables.haar_rotation(dim, 1), tables.fib_codebook(dim, seed=1))
    tq = pk.TurboProfile(dim, 4, tables.rademacher_signs(dim, 1), tables.qjl_matrix(dim, 32, 1), seed=1)
    counts = (C.c_uint64 * 8)()
    L.check(lib.pkv_stats_reset())
    L.check(lib.pkv_stats_read(counts))
    assert list(counts) == [0] * 8
    fib.encode_batch_compact(x)
    L.check(lib.pkv_stats_read(counts))
    blocks = n * dim // 4
    assert 0 < counts[0] < 0.01 * blocks and counts[1] < 1e-3 * blocks and list(counts)[4:] == [0] * 4
    tq.encode_batch_compact(x)
    L.check(lib.pkv_stats_read(counts))
    assert 0 < counts[4] < 0.01 * n * 32 and 0 < counts[5] < 0.05 * n * 32 and 0 < counts[6] < 0.01 * n * 32
    L.check(lib.pkv_stats_reset())
    L.check(lib.pkv_stats_read(counts))
    assert list(counts) == [0] * 8


@pytest.mark.gpu
@pytest.mark.parametrize("dim,bound", [(64, 1.0e-5), (128, 1.7e-5)])
def test_tensor_core_rotation_stays_inside_its_assumed_bound(dim, bound):
    """The bound of the tensor-core tier contains a term assumed for the unit's accumulation rounding
    (PKV_FIB_ROT_ERR_TC / _TC128).  With the capture hook on, the encoder also stores the rotated values as
    the unit delivered them; their distance from the exact rotation (binary64, the reference's (f32) of it)
    must stay inside the bound, with margin."""
    import numpy as np
    import torch
    lib = L.lib()
    n = 60_000
    rot, cb = tables.haar_rotation(dim, 42), tables.fib_codebook(dim, seed=42)
    prof = pk.FibProfile(dim, rot, cb, numerics=L.FIB_NUMERICS_BATCH)
    rng = np.random.default_rng(5)
    x = synthetic_kv(n, dim, seed=31)
    x[: n // 4] = rng.standard_normal((n // 4, dim)).astype(np.float32) * np.float32(1e-4)
    x[n // 4: n // 2, rng.integers(0, dim)] *= np.float32(300.0)   # vectors concentrated in one coordinate
    xd = torch.from_numpy(x).cuda()
    cap = torch.full((n, dim), float("nan"), dtype=torch.float32, device="cuda")
    out = torch.zeros(n * prof.record_bytes, dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    L.check(lib.pkv_test_capture_rotated(cap.data_ptr()))
    try:
        prof.encode_dev(xd.data_ptr(), _flat_layout(1, n, dim), out.data_ptr(), n * prof.record_bytes, err.data_ptr())
        torch.cuda.synchronize()
    finally:
        L.check(lib.pkv_test_capture_rotated(None))
    pk.read_error_word(err.data_ptr())
    got = cap.cpu().numpy()
    assert np.isfinite(got).all()
    x64 = x.astype(np.float64)
    norm = np.sqrt((x64 * x64).sum(1, keepdims=True))
    nrm = (x64 / norm).astype(np.float32).astype(np.float64)          # codec.rs:607-609
    exact = (nrm @ rot.T).astype(np.float32)                           # rotation.rs:104-115, then (f32)
    worst = float(np.abs(got.astype(np.float64) - exact.astype(np.float64)).max())
    print(f"tensor-core rotation d={dim}: largest error {worst:.3e}, bound {bound:.1e}")
    assert worst < 0.5 * bound, worst


@pytest.mark.gpu
@pytest.mark.parametrize("dim", [64, 128])
def test_blocks_at_half_a_codeword_encode_like_the_oracle(oracle_mod, dim):
    """Rotated blocks at half a codeword or halfway to a midpoint of two: the fused scores are near zero there,
    where the certification must rely on the absolute term of its bound."""
    import numpy as np
    n, nb = 8000, dim // 4
    rot, cb = tables.haar_rotation(dim, 42), tables.fib_codebook(dim, seed=42)
    rng = np.random.default_rng(23)
    a, b = rng.integers(0, 32, (n, nb - 1)), rng.integers(0, 32, (n, nb - 1))
    half = 0.5 * cb[a].astype(np.float64) * rng.uniform(0.999999, 1.000001, (n, nb - 1, 1))
    quarter = 0.25 * (cb[a].astype(np.float64) + cb[b].astype(np.float64))
    y = np.where(rng.random((n, nb - 1, 1)) < 0.5, half, quarter)
    rest = np.sqrt(np.maximum(1.0 - (y ** 2).sum((1, 2)), 0.0))
    last = rng.standard_normal((n, 4))
    last *= (rest / np.linalg.norm(last, axis=1))[:, None]
    x = (np.concatenate([y.reshape(n, dim - 4), last], axis=1) @ rot).astype(np.float32)
    for order in (L.ARGMIN_PAIRWISE, L.ARGMIN_SEQUENTIAL):
        prof = pk.FibProfile(dim, rot, cb, argmin_order=order, numerics=L.FIB_NUMERICS_BATCH)
        got = np.frombuffer(prof.encode_batch_compact(x), np.uint8)[L.FB2_HEADER_BYTES:].reshape(n, -1)
        st, want, _, _ = oracle_mod.fib_encode(x, rot, cb, argmin_order=order, numerics=L.FIB_NUMERICS_BATCH, nthreads=4)
        assert st == 0 and np.array_equal(got, want)
