#!/usr/bin/env python
"""Benchmark of the KV-cache codec hot path on B200.

Default workload (``--workload c4``): the two-tier pool on the Qwen2.5-0.5B GQA shape
(24 layers x {K,V} x 2 KV heads x head_dim 64): a 32,768-token shared prefix and 64 agents x 512
unique tokens, every agent's f32 cache holding 32,768 + 64 * 512 = 65,536 positions.  One step =
  1. fib-quant k4_n32 encode of the prefix (FB2 records),
  2. (more than one GPU) all-gather of the FB2 payload so every rank holds the whole cold pool; it runs
     on NCCL's stream beside steps 3 and 4,
  3. turbo-quant b=4 (polar 3 bit + 32 QJL signs, f32 radii) encode of the agents' shells (TQB1),
  4. decode-and-patch of each shell at position n_shared + agent * n_unique of its agent's cache,
  5. decode-and-patch of the pool into every owned agent's cache (one decode, one write per agent).
At N GPUs the agents (shells, caches) are sharded by agent and the prefix encode by layer; the fixed
workload is divided, i.e. strong scaling.  ``--workload c3`` is the same on the SmolLM2-1.7B shape
(800 + 8 x 28 tokens), ``--workload c5`` the Llama-3-8B shape (d = 128, 131,072 + 16 x 2,048 tokens)
sharded by layer and run in groups of 4 layers through the same device buffers.  The single-codec
workloads (c1, c2, ...) time one encoder / decoder pair.

``value`` = f32 KV bytes encoded + f32 KV bytes written into caches, over all ranks, per second of
device time (CUDA events, max over ranks), inputs resident in HBM.  ``value_unique`` counts every
distinct vector once on the decode side.  ``kernels`` gives each kernel's time, algorithmic bytes and
fraction of the measured HBM copy bandwidth and, under ``alu``, the arithmetic ceiling beside it (the
separately rounded binary32 operations the reference's contract fixes per vector, at one per lane and
clock); ``roofline`` repeats the HBM figures for the slowest one.  ``cpu_baseline`` is the oracle on all
host cores, ``cpu_baseline.one_thread`` the same on one.  ``e2e``
is the same step from pinned host buffers: host f32 -> wire blobs on the host through the
``*_encode_batches_compact`` calls, wire bytes back to the device, decode-and-patch into the
device-resident caches, error words read back (the pool's decode-and-patch is launched as soon as its
records are back and runs under the shell encode's transfers).  Data are seeded synthetic tensors with the
configurations' shapes and value distributions; no dataset or checkpoint is read.

With ``--impl reference`` the CPU restatement of the reference (oracle/) runs the same step on a
bounded sample on the host cores instead.
"""
import argparse
import ctypes
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "f32-KV GB/s encode & decode+patch"
SEED = 42
TURBO_PROJ = 32
_C2 = dict(agents=8, layers=24, heads=32, tokens=28, dim=64, cache_tokens=1024, n_shared=800)
WORKLOADS = {
    # the two-tier pool, whole path
    "c4": dict(kind="pool", layers=24, heads=2, dim=64, n_shared=32768, agents=64, n_unique=512, shard="agent",
               layers_per_pass=24, outliers=False,
               desc="C4 two-tier pool, Qwen2.5-0.5B GQA shape 24x{K,V}x2x64: fib k4_n32 prefix of 32768 tokens + "
                    "64 turbo b=4 shells of 512 tokens, decode-and-patch into 64 f32 caches of 65536 positions"),
    "c3": dict(kind="pool", layers=24, heads=32, dim=64, n_shared=800, agents=8, n_unique=28, shard="agent",
               layers_per_pass=24, outliers=False,
               desc="C3 two-tier pool, SmolLM2-1.7B shape 24x{K,V}x32x64: fib k4_n32 prefix of 800 tokens + "
                    "8 turbo b=4 shells of 28 tokens, decode-and-patch into 8 f32 caches of 1024 positions"),
    "c5": dict(kind="pool", layers=32, heads=8, dim=128, n_shared=131072, agents=16, n_unique=2048, shard="layer",
               layers_per_pass=4, outliers=True,
               desc="C5 two-tier pool, Llama-3-8B shape 32x{K,V}x8x128: fib k4_n32 prefix of 131072 tokens + "
                    "16 turbo b=4 shells of 2048 tokens, decode-and-patch into 16 f32 caches, by layer"),
    # single codecs
    "c2": dict(_C2, kind="single", codec="turbo", bits=4, mode=1, lossy=False,
               desc="C2 turbo b=4 (polar 3 bit + 32 QJL, f32 radii) hot shells: 8 agents x 28 tokens, "
                    "SmolLM2-1.7B shape 24x{K,V}x32x64"),
    "c2_lossy": dict(_C2, kind="single", codec="turbo", bits=4, mode=1, lossy=True,
                     desc="C2 turbo b=4 (polar 3 bit + 32 QJL, BlockLogU8 radii), 8 agents x 28 tokens"),
    "c2_polar4": dict(_C2, kind="single", codec="turbo", bits=4, mode=0, lossy=False,
                      desc="C2 turbo polar-only 4-bit angles, f32 radii, 8 agents x 28 tokens"),
    "c1": dict(kind="single", agents=1, layers=24, heads=32, tokens=1024, dim=64, cache_tokens=1024, n_shared=0,
               codec="fib", desc="C1 fib k4_n32 cold tier: 24x{K,V}x32 heads x 1024 tokens x 64"),
    "c1_hadamard": dict(kind="single", agents=1, layers=24, heads=32, tokens=1024, dim=64, cache_tokens=1024,
                        n_shared=0, codec="fib", hadamard=True,
                        desc="C1 with the Walsh-Hadamard rotation of the reference's gpu build on encode (not "
                             "wire-compatible with the stored-matrix pools): 24x{K,V}x32 heads x 1024 tokens x 64"),
    "c5s_fib_hadamard": dict(kind="single", agents=1, layers=32, heads=8, tokens=2048, dim=128, cache_tokens=2048,
                             n_shared=0, codec="fib", hadamard=True,
                             desc="C5 scaled fib prefix with the Walsh-Hadamard rotation on encode: "
                                  "32x{K,V}x8 heads x 2048 tokens x 128"),
    "ops": dict(kind="ops", dim=64, codec="fib",
                desc="the gpu-backend operators on the fib encode path, stand-alone: hadamard_batch in place on "
                     "24x{K,V}x32x1024 vectors of 64 (C1's tensor), on 1,048,576 x 128 and on 131,072 x 1024; "
                     "codebook_lookup_batch (k=4, N=32) on C1's tensor"),
    "c5s_fib": dict(kind="single", agents=1, layers=32, heads=8, tokens=2048, dim=128, cache_tokens=2048,
                    n_shared=0, codec="fib",
                    desc="C5 scaled, fib k4_n32 prefix: 32x{K,V}x8 heads x 2048 tokens x 128"),
    "c5s_turbo": dict(kind="single", agents=4, layers=32, heads=8, tokens=512, dim=128, cache_tokens=1024,
                      n_shared=512, codec="turbo", bits=4, mode=1, lossy=False,
                      desc="C5 scaled, turbo b=4 shells (f32 radii): 4 agents x 512 tokens, 32x{K,V}x8x128"),
    "c5s_turbo_lossy": dict(kind="single", agents=4, layers=32, heads=8, tokens=512, dim=128, cache_tokens=1024,
                            n_shared=512, codec="turbo", bits=4, mode=1, lossy=True,
                            desc="C5 scaled, turbo b=4 shells (BlockLogU8 radii): 4 agents x 512 tokens, 32x{K,V}x8x128"),
}


# ---------------------------------------------------------------------------------------------
# shared helpers
# ---------------------------------------------------------------------------------------------
def alu_roof(kind, d, n_vec, ms, sm_mhz, sms=148):
    """The arithmetic ceiling beside the HBM one: separately rounded binary32 operations the reference's
    contract fixes per vector on the f32 pipe (what runs on the tensor cores is left out), at one operation per
    lane and clock (128 lanes per SM) -> {"f32_ops_per_vector", "roof_ms", "frac"} (frac = roof_ms / ms).
      fib decode      2 d^2          the un-fused multiply and add of every matrix element (rotation.rs:136-149)
      fib encode      11 * 32 * d/4  4 sub, 4 mul, 3 add per (block, codeword) (simd_nearest.rs:24-94); the rotation's
                                     2 d^2 runs on the tensor cores, the norm chain in binary64
      turbo encode    d log2 d + 7 d/2  forward butterflies, per pair 2 mul + add + sqrt + 3 for the residual; the
                                     sketch's 2 m d runs on the tensor cores
      turbo decode    d log2 d + 2 d    two products per pair from the table, butterflies, scale and sign"""
    lg = int(math.log2(d))
    ops = {"fib_decode_patch": 2 * d * d, "fib_encode": 11 * 32 * (d // 4),
           "turbo_encode": d * lg + 7 * (d // 2), "turbo_decode_patch": d * lg + 2 * d}[kind]
    mhz = sm_mhz or 1965.0
    roof_ms = ops * n_vec / (sms * 128 * mhz * 1e6) * 1e3
    return {"f32_ops_per_vector": ops, "roof_ms": roof_ms, "frac": roof_ms / ms if ms > 0 else None,
            "at_sm_mhz": mhz}


def fib_record_bytes(d):
    return 2 + (5 * (d // 4) + 7) // 8


def turbo_record_bytes(d, bits=4, mode=1, lossy=False):
    p = d // 2
    pb = bits - 1 if mode else bits
    return (p + 8 if lossy else 4 * p) + (p * pb + 7) // 8 + (TURBO_PROJ // 8 if mode else 0)


def record_bytes(w):
    if w["codec"] == "fib":
        return fib_record_bytes(w["dim"])
    return turbo_record_bytes(w["dim"], w["bits"], w["mode"], w["lossy"])


def config_dict(w, args):
    """Identical in both arms (ours / reference) for one command line."""
    if w["kind"] == "pool":
        par = (f"{args.gpus} GPU(s): agents (shells, caches) sharded by agent, prefix encode by layer, FB2 payload "
               "all-gathered; no collective inside the codec kernels") if w["shard"] == "agent" else \
              f"{args.gpus} GPU(s): everything sharded by layer, no exchange"
        step = ("fib encode prefix, all-gather FB2 payload (beside the shell chain), turbo encode shells, "
                "decode-and-patch shells, decode-and-patch pool into every agent cache")
    else:
        par = f"{args.gpus} x the same workload (independent replicas)"
        step = "encode every batch, decode-and-patch every batch"
    return {"workload": w["desc"], "step": step, "parallelism": par, "cache_dtype": args.cache_dtype,
            "l2": "inputs larger than L2 (126 MB); single-codec workloads below that size flush L2 with a "
                  "512 MiB write between timed steps"}


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic(key):
    """Per-launch DRAM bytes of a kernel from the committed ncu summary (profiles/dram_traffic.json)."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f).get(key)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
                 "sw_thermal_slowdown": 0x20, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.0005)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_min_mhz": float(np.min(self.samples)),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def synthetic_vectors(n, dim, seed, outliers=False):
    """CPU-side synthetic KV rows with the benchmark distributions."""
    rng = np.random.default_rng(seed)
    z = rng.standard_normal((n, dim)).astype(np.float32)
    if outliers:  # C5: bf16-rounded N(0,1), 1 % of the channels x 20
        z = (z.view(np.uint32) + np.uint32(0x8000) & np.uint32(0xffff0000)).view(np.float32)
        hot = rng.random((64, dim)) < 0.01
        return np.where(hot[np.arange(n) % 64], z * np.float32(20.0), z).astype(np.float32)
    scale = rng.lognormal(0.0, 0.5, size=(64, dim)).astype(np.float32)
    return z * scale[np.arange(n) % 64]


def device_kv(torch, dims, gen, dev, outliers):
    """f32 KV tensor [(agents,) layers, 2, heads, tokens, dim] with the configuration's distribution:
    N(0,1) times a per-(layer, head, channel) log-normal scale, or (C5) bf16-rounded N(0,1) with 1 % of
    the (layer, head, channel) triples scaled by 20."""
    chan = list(dims)
    for i in (-2, -4):  # the same for every token and for K and V
        chan[i] = 1
    if len(dims) == 6:  # ... and for every agent
        chan[0] = 1
    if outliers:
        kv = torch.randn(dims, generator=gen, device=dev).to(torch.bfloat16).to(torch.float32)
        hot = torch.rand(chan, generator=gen, device=dev) < 0.01
        return torch.where(hot, kv * 20.0, kv).contiguous()
    scale = torch.exp(0.5 * torch.randn(chan, generator=gen, device=dev))
    return (torch.randn(dims, generator=gen, device=dev) * scale).contiguous()


def dist_setup(torch):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return rank, world, local, dev


# ---------------------------------------------------------------------------------------------
# CPU side: the oracle as baseline / reference arm
# ---------------------------------------------------------------------------------------------
def cpu_tables(dim):
    from provekv_b200 import tables
    return (tables.haar_rotation(dim, SEED), tables.fib_codebook(dim, seed=SEED),
            tables.rademacher_signs(dim, SEED), tables.qjl_matrix(dim, TURBO_PROJ, SEED))


def cpu_single_rate(w, seconds_budget, nthreads):
    """Oracle encode + decode of a bounded sample of a single-codec workload -> (GB/s, seconds, text)."""
    import oracle
    dim = w["dim"]
    rot, cb, signs, qjl = cpu_tables(dim)
    if w["codec"] == "fib":
        if w.get("hadamard"):
            from provekv_b200 import tables
            rot = tables.hadamard_rotation_matrix(dim, SEED)

        def run(x):
            t0 = time.perf_counter()
            if w.get("hadamard"):
                st, payload, _, _ = oracle.fib_encode_hadamard(x, SEED, cb, nthreads=nthreads)
            else:
                st, payload, _, _ = oracle.fib_encode(x, rot, cb, nthreads=nthreads)
            assert st == 0
            st, _, _, _ = oracle.fib_decode(payload, dim, rot, cb, nthreads=nthreads)
            assert st == 0
            return time.perf_counter() - t0
    else:
        q = qjl if w["mode"] else None
        m, rc = (TURBO_PROJ if w["mode"] else 0), int(w["lossy"])

        def run(x):
            t0 = time.perf_counter()
            st, payload, _, _ = oracle.turbo_encode(x, signs, q, bits=w["bits"], mode=w["mode"], radii_codec=rc,
                                                    libm_mode=oracle.LIBM_PLATFORM, nthreads=nthreads)
            assert st == 0
            st, _, _, _ = oracle.turbo_decode(payload, dim, signs, bits=w["bits"], mode=w["mode"], projections=m,
                                              radii_codec=rc, libm_mode=oracle.LIBM_PLATFORM, nthreads=nthreads)
            assert st == 0
            return time.perf_counter() - t0

    probe = synthetic_vectors(4096 * max(1, nthreads // 4), dim, 1)
    run(probe[:256])
    rate = probe.shape[0] / run(probe)
    total = w["agents"] * w["layers"] * 2 * w["heads"] * w["tokens"]
    n = int(min(total, max(probe.shape[0], rate * seconds_budget)))
    t = run(synthetic_vectors(n, dim, 2))
    return 2 * n * dim * 4 / t / 1e9, t, \
        f"{n} of {total} vectors ({w['codec']} encode + decode, host libm), {nthreads} threads"


def cpu_pool_rate(w, seconds_budget, nthreads):
    """The whole step of a pool workload on a bounded sample, on the host: oracle fib encode + decode of a
    slice of the prefix, oracle turbo encode + decode of a slice of the shells (same proportion as the
    workload), and the patch as one copy of the decoded prefix slice per agent plus one copy of the decoded
    shell slice (the reference patches cache by cache, ppl_validate_multi_agent.py:247-262).
    -> (GB/s in the metric's definition, GB/s counting distinct vectors, seconds, text)."""
    from concurrent.futures import ThreadPoolExecutor

    import oracle
    dim, A = w["dim"], w["agents"]
    rot, cb, signs, qjl = cpu_tables(dim)
    per_tok = w["layers"] * 2 * w["heads"]
    total_p, total_s = per_tok * w["n_shared"], per_tok * w["n_unique"] * A
    ring = [None] * min(A, 4)

    def run(xp, xs):
        t0 = time.perf_counter()
        st, pay_p, _, _ = oracle.fib_encode(xp, rot, cb, nthreads=nthreads)
        assert st == 0
        st, pay_s, _, _ = oracle.turbo_encode(xs, signs, qjl, bits=4, mode=1, radii_codec=0,
                                              libm_mode=oracle.LIBM_PLATFORM, nthreads=nthreads)
        assert st == 0
        st, dec_p, _, _ = oracle.fib_decode(pay_p, dim, rot, cb, nthreads=nthreads)
        assert st == 0
        st, dec_s, _, _ = oracle.turbo_decode(pay_s, dim, signs, bits=4, mode=1, projections=TURBO_PROJ,
                                              radii_codec=0, libm_mode=oracle.LIBM_PLATFORM, nthreads=nthreads)
        assert st == 0
        for i in range(len(ring)):
            if ring[i] is None or ring[i].shape[0] != dec_p.shape[0] + dec_s.shape[0]:
                ring[i] = np.empty((dec_p.shape[0] + dec_s.shape[0], dim), np.float32)

        def patch(a):  # agent a's cache gets the prefix; its own share of the shell slice follows
            dst = ring[a % len(ring)]
            np.copyto(dst[:dec_p.shape[0]], dec_p)
            lo, hi = dec_s.shape[0] * a // A, dec_s.shape[0] * (a + 1) // A
            np.copyto(dst[dec_p.shape[0] + lo:dec_p.shape[0] + hi], dec_s[lo:hi])

        with ThreadPoolExecutor(max(1, min(nthreads, A))) as ex:
            list(ex.map(patch, range(A)))
        return time.perf_counter() - t0

    def sample(n_p):
        n_p = int(max(64, min(total_p, n_p)))
        n_s = int(max(64, min(total_s, round(n_p * total_s / total_p))))
        return synthetic_vectors(n_p, dim, 2, w["outliers"]), synthetic_vectors(n_s, dim, 3, w["outliers"])

    xp, xs = sample(2048 * max(1, nthreads // 4))
    run(xp[:256], xs[:256])
    rate = xp.shape[0] / run(xp, xs)
    xp, xs = sample(rate * seconds_budget)
    t = run(xp, xs)
    n_p, n_s = xp.shape[0], xs.shape[0]
    f32 = dim * 4
    value = ((n_p + n_s) + (A * n_p + n_s)) * f32 / t / 1e9
    unique = 2 * (n_p + n_s) * f32 / t / 1e9
    text = (f"{n_p} of {total_p} prefix vectors and {n_s} of {total_s} shell vectors: oracle fib + turbo encode and "
            f"decode (host libm), prefix patched {A} times, {nthreads} threads")
    return value, unique, t, text


def run_reference(args, w):
    """--impl reference: the CPU restatement of the reference on all host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    budget = min(1.5, 150.0 / max(1, args.steps + args.warmup))
    vals, uniq, times, sample = [], [], [], ""
    for i in range(args.warmup + args.steps):
        if w["kind"] == "pool":
            v, u, t, sample = cpu_pool_rate(w, budget, cores)
        else:
            v, t, sample = cpu_single_rate(w, budget, cores)
            u = v
        if i >= args.warmup:
            vals.append(v)
            uniq.append(u)
            times.append(t)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times) * 1e3),
        "higher_is_better": True, "scaling": "strong" if w["kind"] == "pool" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(w, args),
        "value_unique": float(np.mean(uniq)),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# single-codec workloads (c1, c2, ...): one encoder / decoder pair
# ---------------------------------------------------------------------------------------------
def make_single_profile(w):
    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    if w["codec"] == "fib":
        if w.get("hadamard"):
            from provekv_b200 import tables
            return pk.FibProfile(w["dim"], None, tables.fib_codebook(w["dim"], seed=SEED),
                                 numerics=L.FIB_NUMERICS_BATCH, hadamard_seed=SEED)
        return pk.FibProfile.from_seed(w["dim"], SEED)
    return pk.TurboProfile.from_seed(w["dim"], w["bits"], TURBO_PROJ, SEED, mode=w["mode"],
                                     radii_codec=L.RADII_BLOCK_LOG_U8 if w["lossy"] else L.RADII_F32)


def single_kernel_names(w):
    d = w["dim"]
    if w["codec"] == "fib" and w.get("hadamard"):
        return f"fib_encode_wht_kernel<{d}>", f"fib_decode_patch_kernel<{d}>"
    if w["codec"] == "fib":
        enc = "fib_encode_tc_kernel + fib_encode_fix_kernel<64>" if d == 64 else \
            f"fib_encode_tc128_kernel + fib_encode_fix_kernel<{d}>"
        return enc, f"fib_decode_patch_kernel<{d}>"
    return f"turbo_encode_kernel<{d}>", f"turbo_decode_patch_kernel<{d}>"


def measure_score(torch, w, prof, kv, payload, pstride, n_batches, vpb, flush, steps, dev):
    """Compressed-domain scoring beside the metric (outside its timed region): queries taken from the workload's
    own vectors are prepared on the device, then scored against every record, one query per pass over the
    records and eight queries per pass -> dict for the JSON line's "score" key."""
    d, rec, n_vec = w["dim"], prof.record_bytes, n_batches * vpb
    m = prof.projections if hasattr(prof, "projections") else TURBO_PROJ
    nq = 8
    queries = kv.reshape(-1, d)[:nq].contiguous()
    rot = torch.empty((nq, d), dtype=torch.float32, device=dev)
    proj = torch.empty((nq, max(m, 1)), dtype=torch.float32, device=dev)
    scores = torch.empty((nq, n_vec), dtype=torch.float32, device=dev)
    err = torch.full((1,), -1, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    prof.prepare_queries_dev(queries.data_ptr(), nq, rot.data_ptr(), proj.data_ptr(), err.data_ptr(), stream)
    peak, _ = measured_hbm_peak()
    out = {"records": n_vec, "record_bytes": rec, "queries_prepared_on_device": nq}
    for label, q in (("one_query", 1), ("eight_queries", nq)):
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(steps)]
        for i in range(-3, steps):
            if flush is not None:
                flush.zero_()
            if i >= 0:
                ev[i][0].record()
            prof.score_queries_dev(payload.data_ptr(), pstride, n_batches, vpb, rot.data_ptr(), proj.data_ptr(), q,
                                   scores.data_ptr(), err.data_ptr(), stream)
            if i >= 0:
                ev[i][1].record()
        torch.cuda.synchronize()
        ms = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
        nbytes = (rec + 4 * q) * n_vec
        out[label] = {"ms": ms, "scores_per_s": q * n_vec / (ms * 1e-3), "algorithmic_bytes": nbytes,
                      "achieved_gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / peak}
    assert int(err[0]) == -1, "the score kernel reported a record"
    return out


def measure_single(torch, w, steps, warmup, dev, seed, cache_dtype="f32"):
    """Device-timed encode and decode-and-patch of a single-codec workload -> dict."""
    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    from provekv_b200 import pool
    del pk
    shape = pool.KvShape(w["layers"], w["heads"], w["dim"])
    A, T, d, H = w["agents"], w["tokens"], w["dim"], w["heads"]
    n_vec = shape.vectors(T, A)
    f32_bytes = n_vec * d * 4
    gen = torch.Generator(device=dev).manual_seed(seed)
    kv = device_kv(torch, (A, w["layers"], 2, H, T, d), gen, dev, False)
    prof = make_single_profile(w)
    rec = prof.record_bytes
    assert rec == record_bytes(w)
    big = f32_bytes > (200 << 20)
    vpb, n_batches = T * H, A * w["layers"] * 2
    pstride = pool.payload_batch_stride(vpb, rec)
    payload = torch.empty((n_batches, pstride), dtype=torch.uint8, device=dev)
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[cache_dtype]
    dst = {"f32": L.DST_F32, "f16": L.DST_F16, "bf16": L.DST_BF16}[cache_dtype]
    cache = torch.zeros((A, w["layers"], 2, H, w["cache_tokens"], d), dtype=tdt, device=dev)
    err = torch.full((2,), -1, dtype=torch.int64, device=dev)
    enc_layout = pool.kv_tensor_layout(shape, A, T)
    dec_layout = pool.kv_tensor_layout(shape, A, T, token_capacity=w["cache_tokens"], first_token=w["n_shared"])
    flush = None if big else torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def step(ev=None):
        if ev:
            ev[0].record()
        prof.encode_dev(kv.data_ptr(), enc_layout, payload.data_ptr(), pstride, err.data_ptr(), stream)
        if ev:
            ev[1].record()
        prof.decode_patch_dev(payload.data_ptr(), pstride, dec_layout, cache.data_ptr(), err[1:].data_ptr(), stream,
                              dst_dtype=dst)
        if ev:
            ev[2].record()

    for _ in range(max(warmup, 3)):
        if flush is not None:
            flush.zero_()
        step()
    torch.cuda.synchronize()
    assert int(err[0]) == -1 and int(err[1]) == -1, "a kernel reported a vector error"
    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    launches0 = L.lib().pkv_launch_count()
    for i in range(steps):
        if flush is not None:
            flush.zero_()  # evict the workload from L2; outside the per-step event bracket
        step(events[i])
    torch.cuda.synchronize()
    enc_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in events]))
    dec_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in events]))
    peak, _ = measured_hbm_peak()
    enc_bytes = (4 * d + rec) * n_vec
    dec_bytes = (rec + d * cache.element_size()) * n_vec
    enc_name, dec_name = single_kernel_names(w)
    launches = int(L.lib().pkv_launch_count() - launches0)  # of the timed region; the scoring below is outside it
    score = measure_score(torch, w, prof, kv, payload, pstride, n_batches, vpb, flush, steps, dev) \
        if w["codec"] == "turbo" else None
    return {
        "score": score,
        "prof": prof, "payload": payload, "pstride": pstride, "n_vec": n_vec, "vpb": vpb, "n_batches": n_batches,
        "rec": rec, "err": err, "kv": kv, "flush": flush, "f32_bytes": f32_bytes, "big": big,
        "launches": launches,
        "enc_ms": enc_ms, "dec_ms": dec_ms, "step_ms": enc_ms + dec_ms,
        "kernels": {
            enc_name: {"ms": enc_ms, "algorithmic_bytes": enc_bytes, "achieved_gbs": enc_bytes / enc_ms / 1e6,
                       "frac_of_measured_hbm": enc_bytes / enc_ms / 1e6 / peak},
            dec_name: {"ms": dec_ms, "algorithmic_bytes": dec_bytes, "achieved_gbs": dec_bytes / dec_ms / 1e6,
                       "frac_of_measured_hbm": dec_bytes / dec_ms / 1e6 / peak},
        },
    }


def run_ops(args, w):
    """Device time of pkv_hadamard_batch_dev and pkv_codebook_lookup_batch_dev (CUDA events, inputs larger than
    L2, resident in HBM), each checked against the oracle on a sample first -> one JSON line."""
    if int(os.environ.get("RANK", "0")) != 0:  # a one-GPU measurement: the other ranks of a torchrun launch leave
        return
    import torch

    import oracle
    from provekv_b200 import _lib as L
    from provekv_b200 import tables
    dev = torch.device("cuda", 0)
    L.check(L.lib().pkv_set_device(0))
    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    peak, peak_kind = measured_hbm_peak()
    gen = torch.Generator(device=dev).manual_seed(SEED)
    clocks = ClockSampler(0)
    clocks.__enter__()
    kernels = {}

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
        for e in ev:
            e[0].record()
            fn()
            e[1].record()
        torch.cuda.synchronize()
        return float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))

    launches0 = lib.pkv_launch_count()
    for n, d in ((24 * 2 * 32 * 1024, 64), (1 << 20, 128), (1 << 17, 1024)):
        x = torch.randn((n, d), generator=gen, device=dev)
        chk = x[:4096].clone()
        L.check(lib.pkv_hadamard_batch_dev(chk.data_ptr(), 4096, d, SEED, stream))
        assert np.array_equal(chk.cpu().numpy().view(np.uint32),
                              oracle.hadamard_batch(x[:4096].cpu().numpy(), SEED).view(np.uint32)), d
        ms = timed(lambda: L.check(lib.pkv_hadamard_batch_dev(x.data_ptr(), n, d, SEED, stream)))
        nbytes = 8 * n * d  # every element read once and written once
        kname = f"hadamard_batch_narrow_kernel<{d // 4}>" if d <= 64 else f"hadamard_batch_kernel<{d // 32}>"
        kernels[f"{kname} ({n} x {d})"] = {
            "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
            "frac_of_measured_hbm": nbytes / ms / 1e6 / peak}
        del x
    n, d = 24 * 2 * 32 * 1024, 64
    x = torch.randn((n, d), generator=gen, device=dev) * 0.125
    cb_h = tables.fib_codebook(d, seed=SEED)
    cb = torch.from_numpy(cb_h).to(dev)
    idx = torch.empty((n, d // 4), dtype=torch.int32, device=dev)
    ms = timed(lambda: L.check(lib.pkv_codebook_lookup_batch_dev(x.data_ptr(), cb.data_ptr(), n, d, 4, 32,
                                                                 idx.data_ptr(), stream)))
    assert np.array_equal(idx[:4096].cpu().numpy().view(np.uint32), oracle.codebook_lookup(x[:4096].cpu().numpy(), cb_h))
    nbytes = (4 * d + d) * n  # f32 in, one u32 per 4-block out
    kernels[f"codebook_lookup_kernel ({n} x {d}, k=4, N=32)"] = {
        "ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / ms / 1e6,
        "frac_of_measured_hbm": nbytes / ms / 1e6 / peak,
        "alu": alu_roof("fib_encode", d, n, ms, None)}
    clocks.__exit__()
    clk = clocks.summary()
    name, k = next(iter(kernels.items()))
    print(json.dumps({
        "metric": METRIC, "value": k["achieved_gbs"] / 2, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": k["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"], "step": "one launch of each operator", "l2": "inputs larger than L2"},
        "kernels": kernels,
        "roofline": {"bound": "hbm", "kernel": name, "achieved": k["achieved_gbs"], "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": k["frac_of_measured_hbm"],
                     "algorithmic_bytes_per_launch": k["algorithmic_bytes"], "traffic": None},
        "gpu_launches": int(lib.pkv_launch_count() - launches0), "clocks": clk}))


def run_single(args, w):
    import torch
    import torch.distributed as dist

    import provekv_b200 as pk
    from provekv_b200 import _lib as L

    rank, world, local, dev = dist_setup(torch)
    L.check(L.lib().pkv_set_device(local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    with ClockSampler(local) as clocks:
        t_wall = time.perf_counter()
        m = measure_single(torch, w, args.steps, args.warmup, dev, SEED + rank, args.cache_dtype)
        barrier()
        t_wall = time.perf_counter() - t_wall
    prof, kind, d, rec = m["prof"], w["codec"], w["dim"], m["rec"]
    n_vec, vpb, n_batches, f32_bytes = m["n_vec"], m["vpb"], m["n_batches"], m["f32_bytes"]

    # end to end through the host-buffer C ABI: pinned host f32 -> wire blobs -> pinned host f32
    blob = (L.FB2_HEADER_BYTES if kind == "fib" else L.TQB1_HEADER_BYTES) + vpb * rec
    x_host = torch.empty((n_batches, vpb, d), dtype=torch.float32).pin_memory()
    x_host.copy_(m["kv"].permute(0, 1, 2, 4, 3, 5).reshape(n_batches, vpb, d))  # reference's gather order
    wire_host = torch.empty((n_batches, blob), dtype=torch.uint8).pin_memory()
    out_host = torch.empty((n_batches, vpb, d), dtype=torch.float32).pin_memory()

    def e2e_step():
        pk.encode_batches_compact(prof, x_host.data_ptr(), n_batches, vpb, wire_host.data_ptr(), wire_host.numel())
        pk.decode_batches_compact(prof, wire_host.data_ptr(), n_batches, vpb, out_host.data_ptr(), out_host.numel())

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps

    times = torch.tensor([m["step_ms"], m["enc_ms"], m["dec_ms"], e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    step_ms, enc_ms, dec_ms, e2e_ms = [float(v) for v in times.tolist()]
    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        total_f32 = 2 * f32_bytes * world
        names = list(m["kernels"])
        dom = names[0] if enc_ms >= dec_ms else names[1]
        k = m["kernels"][dom]
        clk = clocks.summary()
        kinds = (f"{kind}_encode", f"{kind}_decode_patch")
        for nm, kd in zip(names, kinds):
            m["kernels"][nm]["alu"] = alu_roof(kd, d, n_vec, m["kernels"][nm]["ms"], clk.get("sm_mhz"))
        line = {
            "metric": METRIC, "value": total_f32 / (step_ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(w, args),
            "value_unique": total_f32 / (step_ms * 1e-3) / 1e9,
            "kernels": m["kernels"],
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": k["achieved_gbs"], "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": k["frac_of_measured_hbm"],
                         "frac_of_nominal_8000": k["achieved_gbs"] / 8000.0,
                         "algorithmic_bytes_per_launch": k["algorithmic_bytes"],
                         "traffic": ncu_traffic(f"{args.workload}:{dom}")},
            "e2e": {"value": total_f32 / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (f32_bytes + n_batches * vpb * rec) * world,
                    "d2h_bytes_per_step": (f32_bytes + n_batches * vpb * rec) * world,
                    "api": f"pkv_{kind}_{{encode,decode}}_batches_compact, pinned host buffers"},
            "gpu_launches": m["launches"], "clocks": clk,
            "ms_x_sm_mhz": step_ms * clk["sm_mhz"] if clk.get("sm_mhz") else None,
            "wall_ms_timed_region": t_wall * 1e3,
        }
        if m.get("score"):
            line["score"] = m["score"]
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            gbs, _, sample = cpu_single_rate(w, 8.0, cores)
            gbs1, _, sample1 = cpu_single_rate(w, 3.0, 1)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                                    "one_thread": {"value": gbs1, "cores": 1, "sample": sample1}}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# the two-tier pool (c3, c4, c5)
# ---------------------------------------------------------------------------------------------
# order inside a step; the all-gather is launched after the prefix encode and waited for just before the pool decode
PHASES = ("fib_encode", "pool_gather", "turbo_encode", "turbo_decode_patch", "gather_wait", "fib_decode_patch")
NOT_KERNELS = ("pool_gather", "gather_wait")


def pool_kernel_names(d):
    fe = "fib_encode_tc_kernel + fib_encode_fix_kernel<64>" if d == 64 else \
        f"fib_encode_tc128_kernel + fib_encode_fix_kernel<{d}>"
    return {"fib_encode": fe, "turbo_encode": f"turbo_encode_kernel<{d},3,rot> + turbo_encode_fix_kernel<{d}>",
            "fib_decode_patch": f"fib_decode_patch_kernel<{d},f32>",
            "turbo_decode_patch": f"turbo_decode_patch_kernel<{d},3,f32>"}


def run_pool(args, w):
    import torch
    import torch.distributed as dist

    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    from provekv_b200 import dist as pdist
    from provekv_b200 import pool

    rank, world, local, dev = dist_setup(torch)
    lib = L.lib()
    L.check(lib.pkv_set_device(local))
    cpus = pdist.bind_rank_to_gpu_numa(local)

    d, H, A = w["dim"], w["heads"], w["agents"]
    shape = pool.KvShape(w["layers"], H, d)
    full = pool.TwoTierPlan(shape, A, w["n_shared"], w["n_unique"], world, rank, w["shard"])
    # the rank's layers go through the device buffers in groups of `lpp` (all at once unless the
    # configuration is too large for that: C5); the plan below describes one group
    lpp = min(w["layers_per_pass"], len(full.dec_layers))
    if w["shard"] == "agent":
        groups, plan = 1, full
        if shape.num_layers % world:
            raise SystemExit("the layer count must be a multiple of the number of GPUs")
    else:
        if len(full.dec_layers) % lpp:
            raise SystemExit("layers per rank must be a multiple of layers_per_pass")
        groups = len(full.dec_layers) // lpp
        plan = pool.TwoTierPlan(pool.KvShape(lpp, H, d), A, w["n_shared"], w["n_unique"], 1, 0, "layer")
    n_ag, Tcap = len(plan.agents), plan.cache_tokens
    L_enc, L_dec = len(plan.enc_layers), len(plan.dec_layers)

    fib = pk.FibProfile.from_seed(d, SEED)
    turbo = pk.TurboProfile.from_seed(d, 4, TURBO_PROJ, SEED, mode=L.TURBO_POLAR_WITH_QJL, radii_codec=L.RADII_F32)
    rec_f, rec_t = fib.record_bytes, turbo.record_bytes
    assert rec_f == fib_record_bytes(d) and rec_t == turbo_record_bytes(d)

    gen = torch.Generator(device=dev).manual_seed(SEED + rank)
    kv_prefix = device_kv(torch, (L_enc, 2, H, w["n_shared"], d), gen, dev, w["outliers"])
    kv_shells = device_kv(torch, (n_ag, L_dec, 2, H, w["n_unique"], d), gen, dev, w["outliers"])
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[args.cache_dtype]
    dst = {"f32": L.DST_F32, "f16": L.DST_F16, "bf16": L.DST_BF16}[args.cache_dtype]
    caches = torch.zeros((n_ag, L_dec, 2, H, Tcap, d), dtype=tdt, device=dev)
    vpb_p, vpb_s = w["n_shared"] * H, w["n_unique"] * H
    ps_p, ps_s = pool.payload_batch_stride(vpb_p, rec_f), pool.payload_batch_stride(vpb_s, rec_t)
    pay_pool = torch.zeros((L_dec * 2, ps_p), dtype=torch.uint8, device=dev)
    gather = world > 1 and w["shard"] == "agent"
    # with several ranks each encodes its layers into a block of its own, gathered into pay_pool
    pay_local_c = torch.zeros((L_enc * 2, ps_p), dtype=torch.uint8, device=dev) if gather else pay_pool
    pay_shells = torch.zeros((n_ag * L_dec * 2, ps_s), dtype=torch.uint8, device=dev)
    err = torch.full((4,), -1, dtype=torch.int64, device=dev)
    lay_pe, lay_pd = plan.prefix_encode_layout(), plan.prefix_decode_layout()
    lay_se, lay_sd = plan.shell_encode_layout(), plan.shell_decode_layout()
    stream = torch.cuda.current_stream().cuda_stream
    n_p_enc, n_p_dec, n_s = plan.prefix_vectors(plan.enc_layers), plan.prefix_vectors(plan.dec_layers), \
        plan.shell_vectors()
    esz = caches.element_size()

    def step(ev=None):
        for g in range(groups):
            e = ev[g] if ev else None
            if e:
                e[0].record()
            fib.encode_dev(kv_prefix.data_ptr(), lay_pe, pay_local_c.data_ptr(), ps_p, err.data_ptr(), stream)
            if e:
                e[1].record()
            # the all-gather of the pool runs on NCCL's stream beside the whole shell chain; only the pool's
            # decode waits for it
            work = pdist.all_gather_pool(pay_local_c, pay_pool, async_op=True) if gather else None
            if e:
                e[2].record()
            turbo.encode_dev(kv_shells.data_ptr(), lay_se, pay_shells.data_ptr(), ps_s, err[1:].data_ptr(), stream)
            if e:
                e[3].record()
            turbo.decode_patch_dev(pay_shells.data_ptr(), ps_s, lay_sd, caches.data_ptr(), err[3:].data_ptr(),
                                   stream, dst_dtype=dst)
            if e:
                e[4].record()
            if work is not None:
                work.wait()
            if e:
                e[5].record()
            fib.decode_patch_dev(pay_pool.data_ptr(), ps_p, lay_pd, caches.data_ptr(), err[2:].data_ptr(), stream,
                                 dst_dtype=dst)
            if e:
                e[6].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    assert all(int(v) == -1 for v in err.tolist()), f"a kernel reported a vector error: {err.tolist()}"

    gather_ms = 0.0
    if gather:  # the collective on its own (in a step it overlaps the shell encode)
        gev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        for a, b in gev:
            barrier()
            a.record()
            pdist.all_gather_pool(pay_local_c, pay_pool)
            b.record()
        torch.cuda.synchronize()
        gather_ms = float(np.median([a.elapsed_time(b) for a, b in gev]))
    events = [[[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(groups)]
              for _ in range(args.steps)]
    launches0 = lib.pkv_launch_count()
    barrier()
    with ClockSampler(local) as clocks:
        t_wall = time.perf_counter()
        for i in range(args.steps):
            step(events[i])
        barrier()
        t_wall = time.perf_counter() - t_wall
    launches = lib.pkv_launch_count() - launches0
    assert all(int(v) == -1 for v in err.tolist())
    phase_ms = [float(np.mean([sum(g[k].elapsed_time(g[k + 1]) for g in ev) for ev in events])) for k in range(6)]
    step_ms = float(np.mean([sum(g[0].elapsed_time(g[6]) for g in ev) for ev in events]))

    # ---- end to end from pinned host buffers ------------------------------------------------
    host = []

    def pinned(shape_, dtype):
        count = int(np.prod(shape_))
        n = max(16, count * torch.empty((), dtype=dtype).element_size())
        p = ctypes.c_void_p()
        L.check(lib.pkv_host_alloc(ctypes.byref(p), n))
        host.append(p)
        buf = (ctypes.c_uint8 * n).from_address(p.value)
        return torch.frombuffer(buf, dtype=dtype, count=count).reshape(shape_)

    hdr_p, hdr_s = L.FB2_HEADER_BYTES, L.TQB1_HEADER_BYTES
    blob_p, blob_s = hdr_p + vpb_p * rec_f, hdr_s + vpb_s * rec_t
    nb_p, nb_s = L_enc * 2, n_ag * L_dec * 2
    xh_p = pinned((nb_p, vpb_p, d), torch.float32)
    xh_s = pinned((nb_s, vpb_s, d), torch.float32)
    wh_p = pinned((nb_p, blob_p), torch.uint8)
    wh_s = pinned((nb_s, blob_s), torch.uint8)
    st_h = pinned((4,), torch.int64)
    xh_p.copy_(kv_prefix.permute(0, 1, 3, 2, 4).reshape(nb_p, vpb_p, d))  # token-major, head-minor gather order
    xh_s.copy_(kv_shells.permute(0, 1, 2, 4, 3, 5).reshape(nb_s, vpb_s, d))
    torch.cuda.synchronize()

    side = torch.cuda.Stream(device=dev)

    def e2e_step():
        # The pool's decode-and-patch is launched as soon as its records are back on the device, so it
        # runs under the host<->device traffic of the shell encode; the shells follow on a second stream
        # (the two decodes write disjoint cache positions).
        for _ in range(groups):
            pk.encode_batches_compact(fib, xh_p.data_ptr(), nb_p, vpb_p, wh_p.data_ptr(), wh_p.numel())
            # the records (headers stripped) go back to the device; the pool is replicated over NVLink
            L.check(lib.pkv_payload_upload(wh_p.data_ptr(), blob_p, hdr_p, nb_p, vpb_p * rec_f,
                                           pay_local_c.data_ptr(), ps_p, stream))
            if gather:
                pdist.all_gather_pool(pay_local_c, pay_pool)
            fib.decode_patch_dev(pay_pool.data_ptr(), ps_p, lay_pd, caches.data_ptr(), err[2:].data_ptr(), stream,
                                 dst_dtype=dst)
            pk.encode_batches_compact(turbo, xh_s.data_ptr(), nb_s, vpb_s, wh_s.data_ptr(), wh_s.numel())
            L.check(lib.pkv_payload_upload(wh_s.data_ptr(), blob_s, hdr_s, nb_s, vpb_s * rec_t,
                                           pay_shells.data_ptr(), ps_s, side.cuda_stream))
            turbo.decode_patch_dev(pay_shells.data_ptr(), ps_s, lay_sd, caches.data_ptr(), err[3:].data_ptr(),
                                   side.cuda_stream, dst_dtype=dst)
            L.check(lib.pkv_memcpy_d2h(st_h[3:].data_ptr(), err[3:].data_ptr(), 8, side.cuda_stream))
            L.check(lib.pkv_memcpy_d2h(st_h.data_ptr(), err.data_ptr(), 24, stream))
            L.check(lib.pkv_stream_synchronize(stream))
            L.check(lib.pkv_stream_synchronize(side.cuda_stream))
            assert int(st_h[2]) == -1 and int(st_h[3]) == -1

    # copy-only floor of the same step: the bytes the step moves over PCIe and no kernel, host->device
    # on one stream and device->host on another

    def copy_only():
        for _ in range(groups):
            L.check(lib.pkv_memcpy_h2d(kv_prefix.data_ptr(), xh_p.data_ptr(), xh_p.numel() * 4, stream))
            L.check(lib.pkv_memcpy_h2d(kv_shells.data_ptr(), xh_s.data_ptr(), xh_s.numel() * 4, stream))
            L.check(lib.pkv_payload_upload(wh_p.data_ptr(), blob_p, hdr_p, nb_p, vpb_p * rec_f,
                                           pay_local_c.data_ptr(), ps_p, stream))
            L.check(lib.pkv_payload_upload(wh_s.data_ptr(), blob_s, hdr_s, nb_s, vpb_s * rec_t,
                                           pay_shells.data_ptr(), ps_s, stream))
            L.check(lib.pkv_payload_download(pay_local_c.data_ptr(), ps_p, nb_p, vpb_p * rec_f, wh_p.data_ptr(),
                                             blob_p, hdr_p, side.cuda_stream))
            L.check(lib.pkv_payload_download(pay_shells.data_ptr(), ps_s, nb_s, vpb_s * rec_t, wh_s.data_ptr(),
                                             blob_s, hdr_s, side.cuda_stream))
        L.check(lib.pkv_stream_synchronize(stream))
        L.check(lib.pkv_stream_synchronize(side.cuda_stream))

    def wall(fn, n):
        barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        barrier()
        return (time.perf_counter() - t0) * 1e3 / n

    est = (xh_p.numel() + xh_s.numel()) * 4 / 40e9 * groups + step_ms * 1e-3  # seconds per e2e step, roughly
    e2e_steps = int(max(2, min(args.steps, 20, math.ceil(4.0 / est))))
    for _ in range(2):
        e2e_step()
    e2e_ms = wall(e2e_step, e2e_steps)
    copy_ms = None
    if not args.no_copy_probe:  # after the timed steps: it overwrites the device inputs with the host copies
        copy_only()
        copy_ms = wall(copy_only, max(2, e2e_steps // 2))
    h2d = ((xh_p.numel() + xh_s.numel()) * 4 + nb_p * vpb_p * rec_f + nb_s * vpb_s * rec_t) * groups
    d2h = (nb_p * vpb_p * rec_f + nb_s * vpb_s * rec_t + 32) * groups

    t = torch.tensor([step_ms, e2e_ms, copy_ms or 0.0, gather_ms] + phase_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms, e2e_ms, copy_ms_max, gather_ms = [float(v) for v in t[:4].tolist()]
    phase_ms = [float(v) for v in t[4:].tolist()]
    counts = torch.tensor([n_p_enc * groups, n_s * groups, n_p_dec * n_ag * groups, h2d, d2h],
                          dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    tot_p_enc, tot_s, tot_p_patched, h2d_all, d2h_all = [float(v) for v in counts.tolist()]

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        f32 = d * 4
        enc_bytes = (tot_p_enc + tot_s) * f32
        dec_bytes = (tot_p_patched + tot_s) * f32
        uniq_dec = (full.prefix_vectors(range(shape.num_layers)) + tot_s) * f32 if w["shard"] == "agent" else \
            (tot_p_enc + tot_s) * f32
        value = (enc_bytes + dec_bytes) / (step_ms * 1e-3) / 1e9
        names = pool_kernel_names(d)
        # algorithmic bytes of this rank's launches (rank 0 stands for all: the shards are equal)
        algo = {"fib_encode": n_p_enc * (f32 + rec_f) * groups,
                "turbo_encode": n_s * (f32 + rec_t) * groups,
                "fib_decode_patch": n_p_dec * (rec_f + n_ag * d * esz) * groups,
                "turbo_decode_patch": n_s * (rec_t + d * esz) * groups}
        kernels = {}
        for k, ph in enumerate(PHASES):
            if ph in NOT_KERNELS:
                continue
            ms = phase_ms[k]
            kernels[names[ph]] = {"ms": ms, "launches_per_step": groups * (2 if ph in ("fib_encode", "turbo_encode") else 1),
                                  "algorithmic_bytes": algo[ph], "achieved_gbs": algo[ph] / ms / 1e6,
                                  "frac_of_measured_hbm": algo[ph] / ms / 1e6 / peak}
        dom_phase = max((ph for ph in PHASES if ph not in NOT_KERNELS), key=lambda ph: phase_ms[PHASES.index(ph)])
        dom = kernels[names[dom_phase]]
        clk = clocks.summary()
        per_rank = {"fib_encode": n_p_enc * groups, "turbo_encode": n_s * groups,
                    "fib_decode_patch": n_p_dec * groups, "turbo_decode_patch": n_s * groups}
        for ph, nv_ph in per_rank.items():  # decode-and-patch: one decode per vector whatever the replica count
            kernels[names[ph]]["alu"] = alu_roof(ph, d, nv_ph, kernels[names[ph]]["ms"], clk.get("sm_mhz"))
        gather_bytes = pay_pool.numel() * groups if gather else 0
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(w, args),
            "value_unique": (enc_bytes + uniq_dec) / (step_ms * 1e-3) / 1e9,
            "encode_gbs": enc_bytes / ((phase_ms[0] + phase_ms[2]) * 1e-3) / 1e9,
            "decode_patch_gbs": dec_bytes / ((phase_ms[3] + phase_ms[5]) * 1e-3) / 1e9,
            "f32_bytes_encoded_per_step": enc_bytes, "f32_bytes_patched_per_step": dec_bytes,
            "kernels": kernels,
            "broadcast_ms": gather_ms,
            "broadcast": {"what": "all-gather of the FB2 payload into every rank's HBM (NCCL), timed on its own; inside "
                                  "a step it runs beside the shell encode and decode, and gather_wait_ms is what the "
                                  "pool decode still waits for" if gather else "none",
                          "gather_wait_ms": phase_ms[PHASES.index("gather_wait")] if gather else 0.0,
                          "bytes_per_rank": gather_bytes,
                          "bus_gbs": (gather_bytes * (world - 1) / world) / (gather_ms * 1e-3) / 1e9
                          if gather and gather_ms > 0 else None},
            "roofline": {"bound": "hbm", "kernel": names[dom_phase], "achieved": dom["achieved_gbs"], "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": dom["frac_of_measured_hbm"],
                         "frac_of_nominal_8000": dom["achieved_gbs"] / 8000.0,
                         "algorithmic_bytes_per_launch": dom["algorithmic_bytes"] / groups,
                         "traffic": ncu_traffic(f"{args.workload}@{world}:{names[dom_phase]}")},
            "e2e": {"value": (enc_bytes + dec_bytes) / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "steps": e2e_steps, "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
                    "copy_only_ms": copy_ms_max if copy_ms is not None else None,
                    "host_cpus_bound": len(cpus),
                    "api": "pinned host f32 -> pkv_{fib,turbo}_encode_batches_compact -> wire blobs on the host -> "
                           "records to the device -> pkv_{fib,turbo}_decode_patch_dev into the device caches -> "
                           "error words to the host; the pool's decode-and-patch runs under the shell encode's "
                           "transfers (second stream)"},
            "gpu_launches": int(launches), "clocks": clk,
            "ms_x_sm_mhz": step_ms * clk["sm_mhz"] if clk.get("sm_mhz") else None,
            "wall_ms_timed_region": t_wall * 1e3,
        }
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            v, u, _, sample = cpu_pool_rate(w, 10.0, cores)
            v1, u1, _, sample1 = cpu_pool_rate(w, 3.0, 1)
            line["cpu_baseline"] = {"value": v, "value_unique": u, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": sample,
                                    "one_thread": {"value": v1, "value_unique": u1, "cores": 1, "sample": sample1}}
        if world == 1 and not args.no_c2:
            caches = kv_prefix = kv_shells = None  # the closures above hold the names, not the tensors
            torch.cuda.empty_cache()
            m = measure_single(torch, WORKLOADS["c2"], 20, 5, dev, SEED)
            line["c2"] = {"workload": WORKLOADS["c2"]["desc"], "encode_ms": m["enc_ms"], "decode_patch_ms": m["dec_ms"],
                          "value": 2 * m["f32_bytes"] / (m["step_ms"] * 1e-3) / 1e9, "kernels": m["kernels"],
                          "l2": "flushed between timed steps"}
        print(json.dumps(line))
    for p in host:
        lib.pkv_host_free(p)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--cache-dtype", default="f32", choices=["f32", "f16", "bf16"],
                    help="element type of the caches decode-and-patch writes (the roofline counts the bytes "
                         "actually written)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c2", action="store_true", help="skip the extra C2 (turbo shells only) measurement")
    ap.add_argument("--no-copy-probe", action="store_true")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    elif w["kind"] == "pool":
        run_pool(args, w)
    elif w["kind"] == "ops":
        run_ops(args, w)
    else:
        run_single(args, w)


if __name__ == "__main__":
    main()
