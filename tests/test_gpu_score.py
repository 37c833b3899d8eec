"""Compressed-domain scoring (TurboQuantizer::score_batch_prepared, turbo-quant/src/turbo.rs:340-381):
the kernel reads wire records and must return the oracle's binary32 scores bit for bit."""
import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import pool, tables

from kvgen import synthetic_kv

pytestmark = pytest.mark.gpu
SEED = 42
CASES = [  # bits, mode, projections, radii codec
    (4, L.TURBO_POLAR_WITH_QJL, 32, L.RADII_F32),
    (4, L.TURBO_POLAR_WITH_QJL, 32, L.RADII_BLOCK_LOG_U8),
    (4, L.TURBO_POLAR_ONLY, 0, L.RADII_F32),
    (8, L.TURBO_POLAR_WITH_QJL, 64, L.RADII_F32),
]


def _tables(dim, m):
    return tables.rademacher_signs(dim, SEED), (tables.qjl_matrix(dim, m, SEED) if m else None)


def _score_on_gpu(prof, payload, n_batches, vpb, rotated, projected):
    import torch
    rec = prof.record_bytes
    stride = pool.payload_batch_stride(vpb, rec)
    host = np.zeros((n_batches, stride), np.uint8)
    host[:, :vpb * rec] = payload.reshape(n_batches, vpb * rec)
    dev = torch.from_numpy(host).cuda()
    rq = torch.from_numpy(rotated).cuda()
    pq = torch.from_numpy(projected if projected.size else np.zeros(1, np.float32)).cuda()
    scores = torch.full((n_batches * vpb,), 123.0, dtype=torch.float32, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.score_dev(dev.data_ptr(), stride, n_batches, vpb, rq.data_ptr(), pq.data_ptr(), scores.data_ptr(),
                   err.data_ptr())
    return scores, err


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("n_batches,vpb", [(1, 1), (3, 129), (2, 1500)])
def test_scores_match_oracle_bits(oracle_mod, dim, case, n_batches, vpb):
    bits, mode, m, rc = case
    signs, qjl = _tables(dim, m)
    n = n_batches * vpb
    x = synthetic_kv(n, dim, seed=n + bits)
    query = synthetic_kv(1, dim, seed=7)[0]
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=bits, mode=mode, radii_codec=rc,
                                               libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    prof = pk.TurboProfile(dim, bits, signs, qjl, mode=mode, radii_codec=rc, seed=SEED)
    rotated, projected = prof.prepare_query(query)
    st, r_ref, p_ref = oracle_mod.turbo_prepare_query(query, signs, qjl)
    assert st == 0 and np.array_equal(rotated.view(np.uint32), r_ref.view(np.uint32))
    assert np.array_equal(projected.view(np.uint32), p_ref.view(np.uint32))
    st, want, _, _ = oracle_mod.turbo_score(payload, dim, rotated, projected, bits=bits, mode=mode, projections=m,
                                           radii_codec=rc, libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    scores, err = _score_on_gpu(prof, payload, n_batches, vpb, rotated, projected)
    pk.read_error_word(err.data_ptr())
    assert np.array_equal(scores.cpu().numpy().view(np.uint32), want.view(np.uint32))
    if mode == L.TURBO_POLAR_ONLY:  # the polar estimate is the inner product with the reconstruction
        st, dec, _, _ = oracle_mod.turbo_decode(payload, dim, signs, bits=bits, mode=mode, projections=m, radii_codec=rc)
        assert np.allclose(want, dec @ query, rtol=1e-4, atol=1e-3)


def test_score_reports_the_first_malformed_record(oracle_mod):
    dim, n = 64, 300
    signs, qjl = _tables(dim, 32)
    x = synthetic_kv(n, dim, seed=3)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=4, mode=1, radii_codec=0)
    payload = payload.copy().reshape(n, -1)
    payload[57, 4:8] = np.frombuffer(np.float32(-1.0).tobytes(), np.uint8)  # a negative radius
    payload[200, 0:4] = np.frombuffer(np.float32(np.inf).tobytes(), np.uint8)
    prof = pk.TurboProfile(dim, 4, signs, qjl, seed=SEED)
    rotated, projected = prof.prepare_query(synthetic_kv(1, dim, seed=8)[0])
    st, _, code, idx = oracle_mod.turbo_score(payload, dim, rotated, projected)
    assert (code, idx) == (L.VEC_BAD_RADIUS, 57)
    _, err = _score_on_gpu(prof, payload, 1, n, rotated, projected)
    with pytest.raises(pk.PkvError) as e:
        pk.read_error_word(err.data_ptr())
    assert e.value.status == L.VEC_BAD_RADIUS and e.value.vector_index == 57


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("n_queries", [1, 3, 8, 11])
def test_queries_prepared_and_scored_on_the_device(oracle_mod, dim, case, n_queries):
    """Queries that live on the device: prepare_query there (bits of the oracle's rotated / projected
    query), then all of them against the records in shared passes (bits of the oracle's scores, query by query)."""
    import torch
    bits, mode, m, rc = case
    signs, qjl = _tables(dim, m)
    n_batches, vpb = 2, 333
    n = n_batches * vpb
    x = synthetic_kv(n, dim, seed=n + bits + n_queries)
    queries = synthetic_kv(n_queries, dim, seed=70 + n_queries)
    st, payload, _, _ = oracle_mod.turbo_encode(x, signs, qjl, bits=bits, mode=mode, radii_codec=rc,
                                               libm_mode=oracle_mod.LIBM_PORTABLE)
    assert st == 0
    prof = pk.TurboProfile(dim, bits, signs, qjl, mode=mode, radii_codec=rc, seed=SEED)
    qd = torch.from_numpy(queries).cuda()
    rot = torch.full((n_queries, dim), 7.0, dtype=torch.float32, device="cuda")
    proj = torch.full((n_queries, max(m, 1)), 7.0, dtype=torch.float32, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.prepare_queries_dev(qd.data_ptr(), n_queries, rot.data_ptr(), proj.data_ptr(), err.data_ptr())
    pk.read_error_word(err.data_ptr())
    rec = prof.record_bytes
    stride = pool.payload_batch_stride(vpb, rec)
    host = np.zeros((n_batches, stride), np.uint8)
    host[:, :vpb * rec] = payload.reshape(n_batches, vpb * rec)
    dev = torch.from_numpy(host).cuda()
    scores = torch.full((n_queries, n), 123.0, dtype=torch.float32, device="cuda")
    prof.score_queries_dev(dev.data_ptr(), stride, n_batches, vpb, rot.data_ptr(), proj.data_ptr(), n_queries,
                           scores.data_ptr(), err.data_ptr())
    pk.read_error_word(err.data_ptr())
    rot_h, proj_h, got = rot.cpu().numpy(), proj.cpu().numpy(), scores.cpu().numpy()
    for q in range(n_queries):
        st, r_ref, p_ref = oracle_mod.turbo_prepare_query(queries[q], signs, qjl)
        assert st == 0 and np.array_equal(rot_h[q].view(np.uint32), r_ref.view(np.uint32)), q
        if m:
            assert np.array_equal(proj_h[q, :m].view(np.uint32), p_ref.view(np.uint32)), q
        st, want, _, _ = oracle_mod.turbo_score(payload, dim, r_ref, p_ref, bits=bits, mode=mode, projections=m,
                                               radii_codec=rc, libm_mode=oracle_mod.LIBM_PORTABLE)
        assert st == 0 and np.array_equal(got[q].view(np.uint32), want.view(np.uint32)), q


def test_a_query_that_is_not_finite_is_reported_by_its_index():
    import torch
    dim = 64
    signs, qjl = _tables(dim, 32)
    prof = pk.TurboProfile(dim, 4, signs, qjl, seed=SEED)
    queries = synthetic_kv(5, dim, seed=1)
    queries[3, 17] = np.inf
    qd = torch.from_numpy(queries).cuda()
    rot = torch.zeros((5, dim), dtype=torch.float32, device="cuda")
    proj = torch.zeros((5, 32), dtype=torch.float32, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    prof.prepare_queries_dev(qd.data_ptr(), 5, rot.data_ptr(), proj.data_ptr(), err.data_ptr())
    with pytest.raises(pk.PkvError) as e:
        pk.read_error_word(err.data_ptr())
    assert e.value.status == L.VEC_NONFINITE_INPUT and e.value.vector_index == 3
