"""Parity report: for each configuration of the codec path (at full size where the CPU oracle finishes
in seconds, scaled down and said so otherwise) encode on the GPU, compare every record byte with the
oracle, decode-and-patch on the GPU and compare the f32 output with the oracle's decode.

    python tests/parity_report.py            # prints a markdown table (needs a B200 and the built oracle)

Inputs are seeded synthetic tensors with the shapes and value distributions of the configurations
(no model captures or datasets are involved)."""
import ctypes as C
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle as oracle_mod  # noqa: E402  (test infrastructure: the checker)
import provekv_b200 as pk  # noqa: E402
from provekv_b200 import _lib as L  # noqa: E402
from provekv_b200 import pool, tables  # noqa: E402

SEED = 42
NTHREADS = os.cpu_count() or 8


def kv_tensor(torch, A, shape, T, seed, outliers=False):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    d = shape.head_dim
    dims = (A, shape.num_layers, 2, shape.num_kv_heads, T, d)
    if outliers:  # C5: N(0,1) in bf16, 1 % of the channels x 20
        kv = torch.randn(dims, generator=gen, device="cuda").to(torch.bfloat16).to(torch.float32)
        hot = torch.rand((1, shape.num_layers, 1, shape.num_kv_heads, 1, d), generator=gen, device="cuda") < 0.01
        kv = torch.where(hot, kv * 20.0, kv)
    else:  # per (layer, head, channel) log-normal scale
        scale = torch.exp(0.5 * torch.randn((1, shape.num_layers, 1, shape.num_kv_heads, 1, d), generator=gen,
                                            device="cuda"))
        kv = torch.randn(dims, generator=gen, device="cuda") * scale
    return kv.contiguous()


def run(torch, name, note, shape, A, T, codec, **kw):
    d = shape.head_dim
    if codec == "fib" and kw.get("hadamard"):
        prof = pk.FibProfile(d, None, tables.fib_codebook(d, seed=SEED), numerics=L.FIB_NUMERICS_BATCH,
                             hadamard_seed=SEED)
    elif codec == "fib":
        prof = pk.FibProfile(d, tables.haar_rotation(d, SEED), tables.fib_codebook(d, seed=SEED))
    else:
        prof = pk.TurboProfile.from_seed(d, kw.get("bits", 4), 32 if kw.get("mode", 1) else 0, SEED,
                                         mode=kw.get("mode", 1),
                                         radii_codec=L.RADII_BLOCK_LOG_U8 if kw.get("lossy") else L.RADII_F32,
                                         libm=L.LIBM_PLATFORM if kw.get("lossy") else L.LIBM_PORTABLE)
    kv = kv_tensor(torch, A, shape, T, seed=kw.get("seed", 0), outliers=kw.get("outliers", False))
    n = kv.numel() // d
    vpb, rec = T * shape.num_kv_heads, prof.record_bytes
    stride = pool.payload_batch_stride(vpb, rec)
    nb = A * shape.num_layers * 2
    payload = torch.zeros((nb, stride), dtype=torch.uint8, device="cuda")
    err = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    lay = pool.kv_tensor_layout(shape, A, T)
    L.check(L.lib().pkv_stats_reset())
    prof.encode_dev(kv.data_ptr(), lay, payload.data_ptr(), stride, err.data_ptr())
    pk.read_error_word(err.data_ptr())
    stats = (C.c_uint64 * 8)()
    L.check(L.lib().pkv_stats_read(stats))
    if codec == "fib":   # blocks settled by the in-kernel exact tier / list entries redone by the exact kernel
        tiers = f"{stats[0]:,} blocks in-kernel, {stats[1]:,} entries to the f64 kernel (of {n * d // 4:,} blocks)"
    else:                # exact atan2f pairs / binary32 re-dots / list entries redone with the reference's sequence
        tiers = (f"{stats[4]:,} pairs exact atan2f (of {n * d // 2:,}), {stats[5]:,} signs re-dotted, "
                 f"{stats[6]:,} entries to the exact kernel (of {n * (32 if kw.get('mode', 1) else 0):,} signs)")
    got = payload[:, :vpb * rec].cpu().numpy().reshape(n, rec)
    gathered = kv.permute(0, 1, 2, 4, 3, 5).reshape(n, d).cpu().numpy()
    t0 = time.perf_counter()
    if codec == "fib" and kw.get("hadamard"):
        st, want, _, _ = oracle_mod.fib_encode_hadamard(gathered, SEED, prof.codebook, nthreads=NTHREADS)
    elif codec == "fib":
        st, want, _, _ = oracle_mod.fib_encode(gathered, prof.rotation, prof.codebook, nthreads=NTHREADS)
    else:
        st, want, _, _ = oracle_mod.turbo_encode(gathered, prof.signs, prof.qjl, bits=kw.get("bits", 4),
                                                 mode=kw.get("mode", 1), radii_codec=prof.radii_codec,
                                                 nthreads=NTHREADS)
    t_cpu = time.perf_counter() - t0
    assert st == 0
    # the same records from the oracle with the host libm (what the Rust reference writes on this machine)
    plat_bytes = "-"
    if codec != "fib":
        st, plat, _, _ = oracle_mod.turbo_encode(gathered, prof.signs, prof.qjl, bits=kw.get("bits", 4),
                                                 mode=kw.get("mode", 1), radii_codec=prof.radii_codec,
                                                 libm_mode=oracle_mod.LIBM_PLATFORM, nthreads=NTHREADS)
        assert st == 0
        plat_bytes = int((got != plat).sum())
        if kw.get("lossy"):
            want = plat  # a LIBM_PLATFORM profile is compared with the host-libm oracle throughout
    bad_bytes = int((got != want).sum())
    out = torch.zeros_like(kv)
    prof.decode_patch_dev(payload.data_ptr(), stride, lay, out.data_ptr(), err.data_ptr())
    pk.read_error_word(err.data_ptr())
    step = max(1, n // 200_000)  # decode compared on a stride-sample of at most ~200k vectors
    dec = out.permute(0, 1, 2, 4, 3, 5).reshape(n, d)[::step].cpu().numpy()
    if codec == "fib":
        st, ref, _, _ = oracle_mod.fib_decode(want[::step], d, prof.rotation, prof.codebook, nthreads=NTHREADS)
    else:
        st, ref, _, _ = oracle_mod.turbo_decode(want[::step], d, prof.signs, bits=kw.get("bits", 4),
                                                mode=kw.get("mode", 1), projections=32 if kw.get("mode", 1) else 0,
                                                radii_codec=prof.radii_codec, nthreads=NTHREADS,
                                                libm_mode=oracle_mod.LIBM_PLATFORM if kw.get("lossy") else
                                                oracle_mod.LIBM_PORTABLE)
    assert st == 0
    diff = np.abs(dec.astype(np.float64) - ref.astype(np.float64))
    bad_words = int((dec.view(np.uint32) != ref.view(np.uint32)).sum())
    rel = float(((out - kv) ** 2).sum() / (kv ** 2).sum())
    print(f"| {name} | {note} | {n:,} | {got.size:,} | {bad_bytes} | {plat_bytes} | {dec.size:,} | {bad_words} | "
          f"{diff.max():.1e} | {rel:.3f} | {tiers} | {t_cpu:.1f} s |", flush=True)
    del kv, out, payload
    torch.cuda.empty_cache()
    return bad_bytes + bad_words


def main():
    import torch
    S, Q, M = pool.SMOLLM2_1_7B, pool.QWEN25_0_5B, pool.LLAMA3_8B
    print("| config | what | vectors | record bytes compared | mismatching bytes | bytes differing from the host-libm "
          "oracle | decoded f32 compared | mismatching words | max abs diff | reconstruction MSE / signal | "
          "flagged by the shortcuts and recomputed | oracle encode time |")
    print("|---|---|---|---|---|---|---|---|---|---|---|---|")
    bad = 0
    bad += run(torch, "C1", "fib k4_n32, 24x2x32x1024x64, full size", S, 1, 1024, "fib")
    bad += run(torch, "C1", "the same vectors through the Walsh-Hadamard rotation of the reference's gpu build "
               "(not wire-compatible with the row above)", S, 1, 1024, "fib", hadamard=True)
    bad += run(torch, "C2", "turbo b=4 (polar 3 + QJL 32), f32 radii, 8 agents x 28 tokens, full size", S, 8, 28, "turbo")
    bad += run(torch, "C2", "same, BlockLogU8 radii, host-libm profile against the host-libm oracle", S, 8, 28, "turbo", lossy=True)
    bad += run(torch, "C2", "turbo polar-only 4-bit angles, f32 radii", S, 8, 28, "turbo", mode=0)
    bad += run(torch, "C3", "fib pool, 800-token prefix, full size", S, 1, 800, "fib", seed=3)
    bad += run(torch, "C4", "fib, d=64, 2 KV heads, prefix 32,768 tokens, full size", Q, 1, 32768, "fib", seed=4)
    bad += run(torch, "C4", "turbo shells, 64 agents x 512 tokens, full size", Q, 64, 512, "turbo", seed=5)
    bad += run(torch, "C5", "fib d=128, 32x2x8 heads, 4,096 of 131,072 tokens (scaled 1/32), bf16 + outlier channels",
               M, 1, 4096, "fib", seed=6, outliers=True)
    bad += run(torch, "C5", "turbo d=128 shells, 16 agents x 256 of 2,048 tokens (scaled 1/8)", M, 16, 256, "turbo",
               seed=7, outliers=True)
    print(f"\ntotal mismatches: {bad}")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
