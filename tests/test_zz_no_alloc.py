"""pkv_fib_encode_dev_static: the fib encoder for callers that may not allocate device memory
on the call path (a serving process whose HBM is fully handed out at start-up, or one running
under an allocator it must not re-enter).  It keeps the encoder's undecided-block list in a fixed
array inside the library image instead of borrowing it from the stream's memory pool.

The test calls it through the C ABI twice in a row on different inputs and checks every record
byte against pkv_fib_encode_dev and against the CPU oracle (so the comparison is not only the
library with itself); the second call also proves that the previous call's leftover list does not
leak into the next one.  The file name sorts last so a `-x` run has already
executed every other test when it gets here.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _layout(L, n_batches, vpb, dim):
    return L.Layout.make(n_batches=(n_batches, 1, 1), batch_stride=(vpb * dim, 0, 0), n_tokens=vpb,
                         n_heads=1, token_stride=dim, head_stride=dim)


@pytest.mark.parametrize("dim", [64, 128])
def test_static_scratch_encode_matches_pool_backed_encode(dim):
    import torch

    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    from provekv_b200 import tables

    import oracle

    lib = L.lib()
    rot, cb = tables.haar_rotation(dim, 7), tables.fib_codebook(dim, seed=7)
    prof = pk.FibProfile(dim, rot, cb)
    rec = prof.record_bytes
    for call, (n_batches, vpb, seed) in enumerate([(5, 3001, 1), (3, 777, 2)]):
        gen = torch.Generator(device="cuda").manual_seed(seed)
        x = torch.randn((n_batches, vpb, dim), generator=gen, device="cuda") * \
            torch.exp(0.5 * torch.randn((1, 1, dim), generator=gen, device="cuda"))
        x = x.contiguous()
        stride = (vpb * rec + 15) // 16 * 16
        want = torch.zeros((n_batches, stride), dtype=torch.uint8, device="cuda")
        got = torch.full((n_batches, stride), 0, dtype=torch.uint8, device="cuda")
        err = torch.full((2,), -1, dtype=torch.int64, device="cuda")
        lay = _layout(L, n_batches, vpb, dim)
        prof.encode_dev(x.data_ptr(), lay, want.data_ptr(), stride, err.data_ptr())
        st = lib.pkv_fib_encode_dev_static(prof.handle, x.data_ptr(), C.byref(lay), got.data_ptr(),
                                           stride, err[1:].data_ptr(), None)
        assert st == L.OK, L.status_string(st)
        torch.cuda.synchronize()
        assert int(err[0]) == -1 and int(err[1]) == -1
        a = want.cpu().numpy()[:, :vpb * rec]
        b = got.cpu().numpy()[:, :vpb * rec]
        assert np.array_equal(a, b), f"call {call}: {(a != b).sum()} differing bytes"
        assert a.any()
        st, ref, _, _ = oracle.fib_encode(x.cpu().numpy().reshape(-1, dim), rot, cb)
        assert st == 0
        ref = ref.reshape(n_batches, vpb * rec)
        assert np.array_equal(b, ref), f"call {call}: {(b != ref).sum()} bytes differ from the oracle"

    # sizes beyond the fixed array are refused with their own status, nothing is launched
    big = L.Layout.make(n_batches=(1, 1, 1), n_tokens=(1 << 20) + 4, n_heads=1, token_stride=dim,
                        head_stride=dim)
    launches = lib.pkv_launch_count()
    st = lib.pkv_fib_encode_dev_static(prof.handle, x.data_ptr(), C.byref(big), got.data_ptr(),
                                       ((1 << 20) + 4) * rec // 16 * 16 + 16, err.data_ptr(), None)
    assert st == L.ERR_STATIC_SCRATCH_TOO_SMALL
    assert "fixed scratch array" in L.status_string(st)
    assert lib.pkv_launch_count() == launches
    # batches below 4 vectors use the reference's single-vector numerics, which this entry lacks
    tiny = _layout(L, 2, 3, dim)
    st = lib.pkv_fib_encode_dev_static(prof.handle, x.data_ptr(), C.byref(tiny), got.data_ptr(), 80,
                                       err.data_ptr(), None)
    assert st == L.ERR_UNSUPPORTED
