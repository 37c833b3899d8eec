"""The kernels' certified shortcuts (provekv_b200/csrc/pkv_fast_paths.h) run on the CPU:
whenever a shortcut declares a decision certain it must equal the exact operation sequence,
including for pairs placed within nano-radians of a sector boundary."""
import ctypes as C

import pytest


def _counts(fn, *args):
    out = (C.c_int64 * 3)()
    fn(*args, out)
    return list(out)


@pytest.mark.parametrize("polar_bits", [2, 3, 4, 7, 8])
@pytest.mark.parametrize("spread", [1e-3, 3e-5, 1e-6, 1e-8])
def test_bucket_shortcut_never_decides_wrong(oracle_mod, polar_bits, spread):
    fn = oracle_mod.lib().pkvo_fast_bucket_check
    fn.argtypes = [C.c_int, C.c_int64, C.c_uint64, C.c_double, C.POINTER(C.c_int64)]
    wrong, undecided, decided = _counts(fn, polar_bits, 400_000, polar_bits * 17 + 1, spread)
    assert wrong == 0
    assert decided > 100_000          # the shortcut carries the bulk of ordinary pairs
    if spread <= 1e-6:
        assert undecided > 150_000    # boundary-hugging pairs are all sent to the exact path


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("scale", [1.0, 1e-3, 1e15, 1e-15])
def test_qjl_sign_shortcut_never_decides_wrong(oracle_mod, dim, scale):
    fn = oracle_mod.lib().pkvo_fast_qjl_check
    fn.argtypes = [C.c_int, C.c_int64, C.c_uint64, C.c_double, C.POINTER(C.c_int64)]
    wrong, undecided, decided = _counts(fn, dim, 200_000, dim + 3, scale)
    assert wrong == 0
    assert decided >= 99_000          # ordinary residuals are decided by the fused dot
    assert undecided >= 50_000        # near-orthogonal ones are not


@pytest.mark.parametrize("spread", [6.0, 1.0, 1e-2, 1e-5, 0.0])
def test_radius_code_shortcut_never_decides_wrong(oracle_mod, spread):
    fn = oracle_mod.lib().pkvo_fast_radius_code_check
    fn.argtypes = [C.c_int64, C.c_uint64, C.c_double, C.POINTER(C.c_int64)]
    wrong, undecided, decided = _counts(fn, 20_000, 11, spread)
    assert wrong == 0
    if spread >= 1.0:
        assert decided > 0.99 * (decided + undecided)   # ordinary blocks: the fast logarithm decides
    if spread <= 1e-5:
        assert decided == 0                             # degenerate span: always the exact path


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("variant", [0, 1])  # operand shortening by truncation / by rounding
@pytest.mark.parametrize("scale", [1.0, 1e-3, 1e15, 1e-15])
def test_qjl_tf32_tier_never_decides_wrong(oracle_mod, dim, variant, scale):
    fn = oracle_mod.lib().pkvo_fast_qjl_tf32_check
    fn.argtypes = [C.c_int, C.c_int64, C.c_uint64, C.c_double, C.c_int, C.POINTER(C.c_int64)]
    wrong, undecided, decided = _counts(fn, dim, 400_000, dim + 5, scale, variant)
    assert wrong == 0
    assert decided >= 190_000         # ordinary residuals: ~98.6 % decided on the tensor cores
    assert undecided >= 20_000        # dots near the threshold go on to the binary32 tier


@pytest.mark.parametrize("check", ["pkvo_fib_fast_check", "pkvo_fib_tc_check"])
@pytest.mark.parametrize("dim,order", [(64, 0), (64, 1), (128, 0)])
def test_fib_rotation_shortcuts_never_decide_wrong(oracle_mod, check, dim, order):
    """Binary32 fused rotation and the emulated three-product TF32 rotation, each with its own
    error bound for the dimension, against the exact f64 sequence: every certified block has the
    reference's index."""
    import numpy as np
    from kvgen import synthetic_kv
    from provekv_b200 import tables
    n = 6000 if dim == 64 else 2500
    rot = np.ascontiguousarray(tables.haar_rotation(dim, 42), dtype=np.float64)
    cb = np.ascontiguousarray(tables.fib_codebook(dim, seed=42), dtype=np.float32)
    x = np.ascontiguousarray(synthetic_kv(n, dim, seed=5), dtype=np.float32)
    fn = getattr(oracle_mod.lib(), check)
    fn.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                   C.POINTER(C.c_int64)]
    out = (C.c_int64 * 6)()
    fn(x.ctypes.data, n, dim, rot.ctypes.data, cb.ctypes.data, 32, order, out)
    wrong, flagged, decided, quot_wrong, quot_uncertain, worst_e9 = list(out)
    blocks = dim // 4
    assert wrong == 0 and quot_wrong == 0
    assert decided + flagged == n * blocks
    assert flagged < 0.008 * n * blocks      # a few per mille of the blocks go to the next tier
    bound = (dim + 3) * 5.97e-8 if check.endswith("fast_check") else (1.0e-5 if dim == 64 else 1.7e-5)
    assert worst_e9 * 1e-9 < bound
    print(check, dim, "flagged share", flagged / (n * blocks), "worst", worst_e9 * 1e-9)


@pytest.mark.parametrize("mode,min_unsure,max_unsure", [(0, 1, 200), (5, 4_000_000, 4_000_000), (9, 1_000_000, 3_900_000),
                                                        (12, 100_000, 600_000), (16, 5_000, 60_000)])
def test_pair_form_normalised_element_is_never_certain_and_wrong(oracle_mod, mode, min_unsure, max_unsure):
    """The binary32 pair form of x / norm against the reference's (f32)((f64)x / norm): random
    arguments (mode 0) and quotients within 2^(mode-52) of a binary32 rounding boundary.  A result
    declared certain must have the division's bits; next to a boundary nothing may be certain, and the
    unsure share must fall off once the distance exceeds the slack of 2^-44."""
    fn = oracle_mod.lib().pkvo_fib_quotient_check
    fn.argtypes = [C.c_uint64, C.c_int64, C.c_int, C.POINTER(C.c_int64)]
    out = (C.c_int64 * 3)()
    fn(2024 + mode, 4_000_000, mode, out)
    wrong, unsure, tested = list(out)
    assert tested == 4_000_000 and wrong == 0
    assert min_unsure <= unsure <= max_unsure


@pytest.mark.parametrize("order", [0, 1])
@pytest.mark.parametrize("n_codewords,scale", [(32, 1.0), (21, 1.0), (32, 3.7), (6, 0.04)])
def test_biased_key_search_never_decides_wrong(oracle_mod, order, n_codewords, scale):
    """The integer-key score search of the Hadamard encoder: typical blocks of unit vectors, blocks of norm
    one (a vector concentrated in one block), and blocks placed on or a few units in the last place beside the
    bisector of two codewords.  No certified block may differ from the reference's scan, and no score may
    leave the binade the keys are ordered in."""
    import numpy as np
    from provekv_b200 import tables
    cb = np.ascontiguousarray(tables.fib_codebook(64, 4, n_codewords, 42, 512, 2, 4) * np.float32(scale), np.float32)
    rng = np.random.default_rng(7 + n_codewords)
    n = 200_000
    typical = rng.standard_normal((n, 4)).astype(np.float32) * np.float32(0.125)
    full = rng.standard_normal((n // 4, 4))
    full = (full / np.linalg.norm(full, axis=1, keepdims=True) * rng.choice([1.0, 0.999, 0.5], (n // 4, 1))).astype(np.float32)
    a, b = rng.integers(0, n_codewords, n), rng.integers(0, n_codewords, n)
    mid = 0.5 * (cb[a].astype(np.float64) + cb[b].astype(np.float64))
    mid += rng.choice([0.0, 1e-8, 1e-7, 1e-6], (n, 1)) * rng.standard_normal((n, 4))
    mid = mid.astype(np.float32)
    mid = mid[np.linalg.norm(mid, axis=1) <= 1.0]
    # scores near zero (|c|^2 = 2 s.c): s = c / 2, and the point halfway to a bisector point
    half = np.concatenate([0.5 * cb[a[:20000]].astype(np.float64) * rng.uniform(0.999999, 1.000001, (20000, 1)),
                           0.25 * (cb[a[:20000]].astype(np.float64) + cb[b[:20000]].astype(np.float64))]).astype(np.float32)
    half = half[np.linalg.norm(half, axis=1) <= 1.0]
    y = np.ascontiguousarray(np.concatenate([typical, full, mid, half]), np.float32)
    fn = oracle_mod.lib().pkvo_fib_biased_search_check
    fn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64)]
    out = (C.c_int64 * 5)()
    assert fn(y.ctypes.data, y.shape[0], cb.ctypes.data, n_codewords, order, out) == 0
    wrong, undecided, certain, by_gap, out_of_binade = list(out)
    assert wrong == 0 and out_of_binade == 0
    assert certain + undecided == y.shape[0]
    assert by_gap > 0.98 * (typical.shape[0] + full.shape[0])      # the quick test settles ordinary blocks
    assert undecided > 0.2 * mid.shape[0]                           # and the bisector cases do reach the exact tier
    print(n_codewords, scale, "undecided", undecided / y.shape[0], "by gap", by_gap / y.shape[0])


@pytest.mark.parametrize("check", ["pkvo_fib_fast_check", "pkvo_fib_tc_check"])
def test_fib_rotation_shortcuts_with_scores_near_zero(oracle_mod, check):
    """Unit vectors whose rotated blocks sit at half a codeword (that codeword's score |c|^2/2 - s.c is ~0, so a
    bound relative to the score alone would not cover the roundings of the fused evaluation) or halfway to
    the midpoint of two codewords; one block carries the rest of the norm.  No certified block may be wrong."""
    import numpy as np
    from provekv_b200 import tables
    dim, n = 64, 6000
    rot = np.ascontiguousarray(tables.haar_rotation(dim, 42), dtype=np.float64)
    cb = np.ascontiguousarray(tables.fib_codebook(dim, seed=42), dtype=np.float32)
    rng = np.random.default_rng(17)
    a, b = rng.integers(0, 32, (n, 15)), rng.integers(0, 32, (n, 15))
    half = 0.5 * cb[a].astype(np.float64) * rng.uniform(0.999999, 1.000001, (n, 15, 1))
    quarter = 0.25 * (cb[a].astype(np.float64) + cb[b].astype(np.float64))
    y = np.where(rng.random((n, 15, 1)) < 0.5, half, quarter)
    rest = np.sqrt(np.maximum(1.0 - (y ** 2).sum((1, 2)), 0.0))            # the 16th block completes the unit norm
    last = rng.standard_normal((n, 4))
    last *= (rest / np.linalg.norm(last, axis=1))[:, None]
    yv = np.concatenate([y.reshape(n, 60), last], axis=1)
    x = np.ascontiguousarray((yv @ rot).astype(np.float32))                  # x = M^T y
    fn = getattr(oracle_mod.lib(), check)
    fn.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                   C.POINTER(C.c_int64)]
    for order in (0, 1):
        out = (C.c_int64 * 6)()
        fn(x.ctypes.data, n, dim, rot.ctypes.data, cb.ctypes.data, 32, order, out)
        wrong, flagged, decided, quot_wrong, quot_uncertain, worst_e9 = list(out)
        assert wrong == 0 and quot_wrong == 0 and decided + flagged == n * 16
        assert decided > 0.5 * n * 16
