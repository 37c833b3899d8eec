"""The two gpu-backend operators on the fib encode path as stand-alone device calls
(gpu_backend::hadamard_batch, gpu-backend/src/lib.rs:66-90; codebook_lookup_batch, :196-239) against the
oracle's restatement of the crate's CPU code (fallback.rs:12-62, 254-305), bit for bit."""
import numpy as np
import pytest

from provekv_b200 import _lib as L
from provekv_b200 import tables
from kvgen import synthetic_kv

pytestmark = pytest.mark.gpu


def _hadamard_gpu(x, seed):
    import torch
    d = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()
    L.check(L.lib().pkv_hadamard_batch_dev(d.data_ptr(), x.shape[0], x.shape[1], seed, None))
    torch.cuda.synchronize()
    return d.cpu().numpy()


@pytest.mark.parametrize("dim", [64, 128, 256, 512, 1024, 32, 16, 8, 2, 1, 96, 768, 100, 33, 7])
def test_hadamard_batch_bits(oracle_mod, dim):
    """Powers of two, dims that are padded (96 -> 128, 768 -> 1024, 100, 33, 7) and the sub-warp sizes."""
    seed = 0xDEADBEEF12345678
    for n in (1, 37, 3000):
        rng = np.random.default_rng(dim + n)
        x = (rng.standard_normal((n, dim)) * rng.choice([1e-20, 1.0, 3e5], (n, 1))).astype(np.float32)
        x[0, :] = 0.0
        x[0, 0] = 1.0                                        # the reference's impulse test
        got, want = _hadamard_gpu(x, seed), oracle_mod.hadamard_batch(x, seed)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (dim, n)
    pd = 1 << (dim - 1).bit_length() if dim > 1 else 1
    assert np.all(np.abs(np.abs(got[0]) - 1.0 / np.sqrt(np.float32(pd))) < 1e-6)


def test_hadamard_rows_that_are_not_16_byte_aligned(oracle_mod):
    """A view that starts 4 bytes into an allocation: the scalar access path."""
    import torch
    n, dim, seed = 500, 128, 5
    x = synthetic_kv(n, dim, seed=3)
    buf = torch.zeros(n * dim + 1, dtype=torch.float32, device="cuda")
    buf[1:] = torch.from_numpy(x.reshape(-1)).cuda()
    L.check(L.lib().pkv_hadamard_batch_dev(buf.data_ptr() + 4, n, dim, seed, None))
    got = buf[1:].cpu().numpy().reshape(n, dim)
    assert float(buf[0]) == 0.0
    assert np.array_equal(got.view(np.uint32), oracle_mod.hadamard_batch(x, seed).view(np.uint32))
    assert L.lib().pkv_hadamard_batch_dev(buf.data_ptr(), 1, 2048, seed, None) == L.ERR_UNSUPPORTED


def _lookup_gpu(x, cb):
    import torch
    xd = torch.from_numpy(np.ascontiguousarray(x, np.float32)).cuda()
    cd = torch.from_numpy(np.ascontiguousarray(cb, np.float32)).cuda()
    n, d = x.shape
    out = torch.full((n * (d // 4),), 99, dtype=torch.int32, device="cuda")
    L.check(L.lib().pkv_codebook_lookup_batch_dev(xd.data_ptr(), cd.data_ptr(), n, d, 4, cb.shape[0], out.data_ptr(), None))
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint32).reshape(n, d // 4)


@pytest.mark.parametrize("dim", [64, 128, 4, 20, 96])
@pytest.mark.parametrize("n_codewords", [32, 21, 2, 1])
def test_codebook_lookup_indices(oracle_mod, dim, n_codewords):
    rng = np.random.default_rng(dim * 100 + n_codewords)
    cb = tables.fib_codebook(64, 4, max(n_codewords, 2), 42, 512, 2, 4)[:n_codewords].copy()
    if n_codewords >= 4:
        cb[3] = cb[1]                                         # equal codewords: the scan keeps the lower index
    n = 4000
    x = rng.standard_normal((n, dim)).astype(np.float32) * np.float32(0.2)
    x[:400] *= np.float32(1e6)                                # far from every codeword
    x[400:800] *= np.float32(1e-20)
    blocks = x.reshape(n, dim // 4, 4)
    a, b = rng.integers(0, n_codewords, (600, dim // 4)), rng.integers(0, n_codewords, (600, dim // 4))
    mid = 0.5 * (cb[a].astype(np.float64) + cb[b].astype(np.float64))
    mid += rng.choice([0.0, 1e-8, 3e-7], mid.shape[:2] + (1,)) * rng.standard_normal(mid.shape)
    blocks[800:1400] = mid.astype(np.float32)                 # on and beside the bisector of two codewords
    blocks[1400:1500] = cb[a[:100]]                           # exactly on a codeword
    blocks[1500:1600] = (0.5 * cb[a[:100]].astype(np.float64) * rng.uniform(0.999999, 1.000001, (100, dim // 4, 1))
                         ).astype(np.float32)                 # s = c / 2: |c|^2 = 2 s.c, that codeword's score is ~0
    blocks[1600:1700] = (0.25 * (cb[a[:100]].astype(np.float64) + cb[b[:100]].astype(np.float64))
                         ).astype(np.float32)                 # halfway to a bisector point: two scores near zero
    blocks[1700:1800] = (2.0 * cb[a[:100]].astype(np.float64)).astype(np.float32)
    x = blocks.reshape(n, dim)
    got, want = _lookup_gpu(x, cb), oracle_mod.codebook_lookup(x, cb)
    assert np.array_equal(got, want), np.argwhere(got != want)[:5]


def test_codebook_lookup_with_values_that_are_not_finite(oracle_mod):
    """Distances that are +inf or NaN never win the reference's scan (index 0 when none is below +inf)."""
    cb = tables.fib_codebook(64, seed=42)
    cb2 = cb.copy()
    cb2[0, 0] = np.inf                                        # codeword 0 is infinitely far from everything finite
    x = synthetic_kv(300, 64, seed=4)
    x[5, 0] = np.nan
    x[6, 9] = np.inf
    x[7, :] = 3e38                                            # squares overflow
    x[8, 20:24] = [np.inf, -np.inf, np.nan, 0.0]
    for book in (cb, cb2):
        got, want = _lookup_gpu(x, book), oracle_mod.codebook_lookup(x, book)
        assert np.array_equal(got, want), np.argwhere(got != want)[:5]
    assert L.lib().pkv_codebook_lookup_batch_dev(1 << 20, 1 << 20, 1, 64, 8, 32, 1 << 20, None) == L.ERR_UNSUPPORTED
    assert L.lib().pkv_codebook_lookup_batch_dev(1 << 20, 1 << 20, 1, 66, 4, 32, 1 << 20, None) == L.ERR_INVALID_ARGUMENT
