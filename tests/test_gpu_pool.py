"""The composed two-tier pool on the GPU against the oracle: fib-encode the shared prefix once,
turbo-encode every agent's shell, decode-and-patch both into the agents' caches at the positions of
the reference's patch loop (proveKV/scripts/ppl_validate_multi_agent.py:226-271), driven by the same
TwoTierPlan layouts the benchmark and a multi-GPU deployment use.

C3 runs whole (SmolLM2-1.7B shape, 800 + 8 x 28 tokens, 8 caches of 1024 positions); C4 (Qwen2.5-0.5B
GQA shape, 32768 + 64 x 512 tokens) runs at full size with the agents taken in four blocks of 16, i.e.
the plans of a 4-GPU agent-sharded run executed one after the other on one GPU.
"""
import os

import numpy as np
import pytest

import provekv_b200 as pk
from provekv_b200 import _lib as L
from provekv_b200 import pool, tables

pytestmark = pytest.mark.gpu

SEED = 42
NTHREADS = os.cpu_count() or 8


def _kv(torch, dims, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    chan = list(dims)
    chan[-2] = chan[-4] = 1
    if len(dims) == 6:
        chan[0] = 1
    scale = torch.exp(0.5 * torch.randn(chan, generator=gen, device="cuda"))
    return (torch.randn(dims, generator=gen, device="cuda") * scale).contiguous()


def _run_pool(oracle_mod, shape, A, n_shared, n_unique, world):
    import torch
    d, H, Lyr = shape.head_dim, shape.num_kv_heads, shape.num_layers
    rot, cb = tables.haar_rotation(d, SEED), tables.fib_codebook(d, seed=SEED)
    signs, qjl = tables.rademacher_signs(d, SEED), tables.qjl_matrix(d, 32, SEED)
    fib = pk.FibProfile(d, rot, cb)
    turbo = pk.TurboProfile(d, 4, signs, qjl, seed=SEED)
    rec_f, rec_t = fib.record_bytes, turbo.record_bytes
    vpb_p, vpb_s = n_shared * H, n_unique * H
    ps_p, ps_s = pool.payload_batch_stride(vpb_p, rec_f), pool.payload_batch_stride(vpb_s, rec_t)
    err = torch.full((4,), -1, dtype=torch.int64, device="cuda")

    # the cold pool: every rank's layer block encoded into its place, as the all-gather leaves it
    kv_prefix = _kv(torch, (Lyr, 2, H, n_shared, d), 1)
    pay_pool = torch.zeros((Lyr * 2, ps_p), dtype=torch.uint8, device="cuda")
    for r in range(world):
        plan = pool.TwoTierPlan(shape, A, n_shared, n_unique, world, r, "agent")
        el = plan.enc_layers
        fib.encode_dev(kv_prefix[el.start:el.stop].data_ptr(), plan.prefix_encode_layout(),
                       pay_pool[2 * el.start:2 * el.stop].data_ptr(), ps_p, err.data_ptr())
    pk.read_error_word(err.data_ptr())
    n_p = Lyr * 2 * vpb_p
    st, want_p, _, _ = oracle_mod.fib_encode(kv_prefix.permute(0, 1, 3, 2, 4).reshape(n_p, d).cpu().numpy(), rot, cb,
                                             nthreads=NTHREADS)
    assert st == 0
    got_p = pay_pool[:, :vpb_p * rec_f].cpu().numpy().reshape(n_p, rec_f)
    assert np.array_equal(got_p, want_p), "pool bytes differ from the oracle"
    st, dec_p, _, _ = oracle_mod.fib_decode(want_p, d, rot, cb, nthreads=NTHREADS)
    assert st == 0
    expect_prefix = torch.from_numpy(dec_p.reshape(Lyr, 2, n_shared, H, d)).cuda().permute(0, 1, 3, 2, 4)
    expect_prefix = expect_prefix.contiguous().view(torch.int32)
    del kv_prefix

    Tcap = n_shared + A * n_unique
    for r in range(world):
        plan = pool.TwoTierPlan(shape, A, n_shared, n_unique, world, r, "agent")
        ag = plan.agents
        assert plan.cache_tokens == Tcap
        kv_shells = _kv(torch, (len(ag), Lyr, 2, H, n_unique, d), 100 + r)
        pay_s = torch.zeros((len(ag) * Lyr * 2, ps_s), dtype=torch.uint8, device="cuda")
        turbo.encode_dev(kv_shells.data_ptr(), plan.shell_encode_layout(), pay_s.data_ptr(), ps_s, err[1:].data_ptr())
        pk.read_error_word(err[1:].data_ptr())
        n_s = len(ag) * Lyr * 2 * vpb_s
        st, want_s, _, _ = oracle_mod.turbo_encode(kv_shells.permute(0, 1, 2, 4, 3, 5).reshape(n_s, d).cpu().numpy(),
                                                   signs, qjl, bits=4, mode=1, radii_codec=0,
                                                   libm_mode=oracle_mod.LIBM_PORTABLE, nthreads=NTHREADS)
        assert st == 0
        got_s = pay_s[:, :vpb_s * rec_t].cpu().numpy().reshape(n_s, rec_t)
        assert np.array_equal(got_s, want_s), "shell bytes differ from the oracle"
        st, dec_s, _, _ = oracle_mod.turbo_decode(want_s, d, signs, bits=4, mode=1, projections=32, radii_codec=0,
                                                  libm_mode=oracle_mod.LIBM_PORTABLE, nthreads=NTHREADS)
        assert st == 0
        expect_shell = torch.from_numpy(dec_s.reshape(len(ag), Lyr, 2, n_unique, H, d)).cuda().permute(0, 1, 2, 4, 3, 5)
        del kv_shells

        fill = 7.0
        caches = torch.full((len(ag), Lyr, 2, H, Tcap, d), fill, device="cuda")
        fib.decode_patch_dev(pay_pool.data_ptr(), ps_p, plan.prefix_decode_layout(), caches.data_ptr(),
                             err[2:].data_ptr())
        turbo.decode_patch_dev(pay_s.data_ptr(), ps_s, plan.shell_decode_layout(), caches.data_ptr(),
                               err[3:].data_ptr())
        pk.read_error_word(err[2:].data_ptr())
        pk.read_error_word(err[3:].data_ptr())
        for i, a in enumerate(ag):
            c = caches[i]
            assert torch.equal(c[:, :, :, :n_shared, :].view(torch.int32), expect_prefix), \
                f"agent {a}: prefix differs"
            pos = pool.agent_patch_position(n_shared, n_unique, a)
            assert torch.equal(c[:, :, :, pos:pos + n_unique, :].contiguous().view(torch.int32),
                               expect_shell[i].contiguous().view(torch.int32)), f"agent {a}: shell differs"
            rest = torch.ones(Tcap, dtype=torch.bool, device="cuda")
            rest[:n_shared] = False
            rest[pos:pos + n_unique] = False
            assert bool((c[:, :, :, rest, :] == fill).all()), f"agent {a}: positions outside the patch were written"
        del caches, expect_shell, pay_s
        torch.cuda.empty_cache()


def test_c3_pool_eight_shells_eight_caches(oracle_mod):
    _run_pool(oracle_mod, pool.SMOLLM2_1_7B, 8, 800, 28, world=1)


def test_c3_pool_as_two_agent_shards(oracle_mod):
    _run_pool(oracle_mod, pool.SMOLLM2_1_7B, 8, 800, 28, world=2)


def test_c4_full_size_in_four_agent_blocks(oracle_mod):
    _run_pool(oracle_mod, pool.QWEN25_0_5B, 64, 32768, 512, world=4)
