#!/usr/bin/env python
"""Benchmark of the KV-cache codec hot path on B200.

Workload (``--workload c2``, the configuration the metric is quoted on): the
turbo-quant b=4 hot shells of 8 agents x 28 unique tokens of a SmolLM2-1.7B
shaped cache (24 layers x {K,V} x 32 heads x head_dim 64 = 344,064 vectors,
88.1 MB f32).  A step = encode all 384 (agent, layer, K|V) batches to TQB1
records, then decode-and-patch them into the agents' f32 caches.  Data are
seeded synthetic tensors with the stated distribution (x = z*s, z ~ N(0,1),
s ~ lognormal(0, 0.5) per (layer, head, channel)); no dataset or checkpoint is
read.

``value`` is f32-KV GB/s = (f32 bytes encoded + f32 bytes decoded) / device time,
inputs resident in HBM; L2 is flushed between timed steps (the workload is
smaller than the 126 MB L2).  ``e2e`` is the same quantity through the
host-buffer C-ABI calls, copies included.  ``roofline`` describes the slower of
the two kernels.  With ``--impl reference`` the CPU restatement of the reference
(oracle/) is timed on the host cores instead.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "f32-KV GB/s encode & decode+patch"
SEED = 42
_C2 = dict(agents=8, layers=24, heads=32, tokens=28, dim=64, cache_tokens=1024, n_shared=800)
WORKLOADS = {
    # the configuration the metric is quoted on
    "c2": dict(_C2, codec="turbo", bits=4, mode=1, lossy=False,
               desc="C2 turbo b=4 (polar 3 bit + 32 QJL, f32 radii) hot shells: 8 agents x 28 tokens, "
                    "SmolLM2-1.7B shape 24x{K,V}x32x64"),
    # the other radii codec / the literal 4-bit-angle reading of the same shape
    "c2_lossy": dict(_C2, codec="turbo", bits=4, mode=1, lossy=True,
                     desc="C2 turbo b=4 (polar 3 bit + 32 QJL, BlockLogU8 radii), 8 agents x 28 tokens"),
    "c2_polar4": dict(_C2, codec="turbo", bits=4, mode=0, lossy=False,
                      desc="C2 turbo polar-only 4-bit angles, f32 radii, 8 agents x 28 tokens"),
    # cold tier: one whole SmolLM2-1.7B cache, fib k4_n32
    "c1": dict(agents=1, layers=24, heads=32, tokens=1024, dim=64, cache_tokens=1024, n_shared=0,
               codec="fib", desc="C1 fib k4_n32 cold tier: 24x{K,V}x32 heads x 1024 tokens x 64"),
    # d = 128 (Llama-3-8B shape, 32 layers x 8 KV heads), the long-context configuration cut to a size
    # one launch finishes in milliseconds: 1,048,576 vectors (537 MB f32) per launch
    "c5s_fib": dict(agents=1, layers=32, heads=8, tokens=2048, dim=128, cache_tokens=2048, n_shared=0,
                    codec="fib", desc="C5 scaled, fib k4_n32 prefix: 32x{K,V}x8 heads x 2048 tokens x 128"),
    "c5s_turbo": dict(agents=4, layers=32, heads=8, tokens=512, dim=128, cache_tokens=1024, n_shared=512,
                      codec="turbo", bits=4, mode=1, lossy=False,
                      desc="C5 scaled, turbo b=4 shells (f32 radii): 4 agents x 512 tokens, 32x{K,V}x8x128"),
    "c5s_turbo_lossy": dict(agents=4, layers=32, heads=8, tokens=512, dim=128, cache_tokens=1024, n_shared=512,
                            codec="turbo", bits=4, mode=1, lossy=True,
                            desc="C5 scaled, turbo b=4 shells (BlockLogU8 radii): 4 agents x 512 tokens, 32x{K,V}x8x128"),
}
TURBO_PROJ = 32


def record_bytes(w):
    d, p = w["dim"], w["dim"] // 2
    if w["codec"] == "fib":
        return 2 + (5 * d // 4 + 7) // 8
    pb = w["bits"] - 1 if w["mode"] else w["bits"]
    return (p + 8 if w["lossy"] else 4 * p) + (p * pb + 7) // 8 + (TURBO_PROJ // 8 if w["mode"] else 0)


def algo_bytes_per_vector(w):
    """f32 vector in or out plus its wire record (fib 268 B, turbo 400 / 312 B at d=64)."""
    return 4 * w["dim"] + record_bytes(w)


def make_profile(w):
    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    if w["codec"] == "fib":
        return pk.FibProfile.from_seed(w["dim"], SEED)
    return pk.TurboProfile.from_seed(w["dim"], w["bits"], TURBO_PROJ, SEED, mode=w["mode"],
                                     radii_codec=L.RADII_BLOCK_LOG_U8 if w["lossy"] else L.RADII_F32)


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic(kernel_key):
    """Per-launch DRAM bytes of a kernel from the committed ncu summary, if any."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f).get(kernel_key)
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
            time.sleep(0.005)

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
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def synthetic_vectors(n, dim, seed):
    """CPU-side synthetic KV rows with the benchmark distribution."""
    rng = np.random.default_rng(seed)
    scale = rng.lognormal(0.0, 0.5, size=(64, dim)).astype(np.float32)
    z = rng.standard_normal((n, dim)).astype(np.float32)
    return z * scale[np.arange(n) % 64]


def cpu_codec_rate(w, seconds_budget, nthreads):
    """Time the oracle (turbo encode + decode) on a bounded sample; returns (GB/s, sample text)."""
    import oracle
    from provekv_b200 import tables
    dim = w["dim"]
    if w["codec"] == "fib":
        rot, cb = tables.haar_rotation(dim, SEED), tables.fib_codebook(dim, seed=SEED)

        def run(x):
            t0 = time.perf_counter()
            st, payload, _, _ = oracle.fib_encode(x, rot, cb, nthreads=nthreads)
            assert st == 0
            st, _, _, _ = oracle.fib_decode(payload, dim, rot, cb, nthreads=nthreads)
            assert st == 0
            return time.perf_counter() - t0
    else:
        signs = tables.rademacher_signs(dim, SEED)
        qjl = tables.qjl_matrix(dim, TURBO_PROJ, SEED) if w["mode"] else None
        m, rc = (TURBO_PROJ if w["mode"] else 0), int(w["lossy"])

        def run(x):
            t0 = time.perf_counter()
            st, payload, _, _ = oracle.turbo_encode(x, signs, qjl, bits=w["bits"], mode=w["mode"],
                                                    radii_codec=rc, libm_mode=oracle.LIBM_PLATFORM,
                                                    nthreads=nthreads)
            assert st == 0
            st, _, _, _ = oracle.turbo_decode(payload, dim, signs, bits=w["bits"], mode=w["mode"],
                                              projections=m, radii_codec=rc,
                                              libm_mode=oracle.LIBM_PLATFORM, nthreads=nthreads)
            assert st == 0
            return time.perf_counter() - t0

    probe = synthetic_vectors(4096 * max(1, nthreads // 4), dim, 1)
    run(probe[:256])
    t = run(probe)
    rate = probe.shape[0] / t
    total = w["agents"] * w["layers"] * 2 * w["heads"] * w["tokens"]
    n = int(min(total, max(probe.shape[0], rate * seconds_budget)))
    x = synthetic_vectors(n, dim, 2)
    t = run(x)
    gbs = 2 * n * dim * 4 / t / 1e9
    return gbs, t, f"{n} of {total} vectors ({w['codec']} encode + decode, host libm), {nthreads} threads"


def run_reference(args, w):
    """--impl reference: the CPU restatement of the reference on all host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    budget = min(1.5, 150.0 / max(1, args.steps + args.warmup))
    times, sample, gbs = [], "", 0.0
    for i in range(args.warmup + args.steps):
        gbs, t, sample = cpu_codec_rate(w, budget, cores)
        if i >= args.warmup:
            times.append((gbs, t))
    value = float(np.mean([g for g, _ in times]))
    ms = float(np.mean([t for _, t in times]) * 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["desc"], "step": "bounded sample of the workload per step"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_ours(args, w):
    import torch
    import torch.distributed as dist

    import provekv_b200 as pk
    from provekv_b200 import _lib as L
    from provekv_b200 import pool

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L.check(L.lib().pkv_set_device(local))

    shape = pool.KvShape(w["layers"], w["heads"], w["dim"])
    A, T, d, H = w["agents"], w["tokens"], w["dim"], w["heads"]
    n_vec = shape.vectors(T, A)
    f32_bytes = n_vec * d * 4

    # synthetic KV, resident in HBM: kv[agent][layer][side][head][token][dim]
    gen = torch.Generator(device=dev).manual_seed(SEED + rank)
    scale = torch.exp(0.5 * torch.randn((1, w["layers"], 1, H, 1, d), generator=gen, device=dev))
    kv = torch.randn((A, w["layers"], 2, H, T, d), generator=gen, device=dev) * scale
    kv = kv.contiguous()
    prof = make_profile(w)
    rec = prof.record_bytes
    assert rec == record_bytes(w)
    algo_bytes = algo_bytes_per_vector(w)
    kind = w["codec"]
    big = f32_bytes > (200 << 20)  # larger than L2: no flush needed
    vpb = T * H
    n_batches = A * w["layers"] * 2
    pstride = pool.payload_batch_stride(vpb, rec)
    payload = torch.empty((n_batches, pstride), dtype=torch.uint8, device=dev)
    cache_dtype = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[args.cache_dtype]
    dst = {"f32": L.DST_F32, "f16": L.DST_F16, "bf16": L.DST_BF16}[args.cache_dtype]
    cache = torch.zeros((A, w["layers"], 2, H, w["cache_tokens"], d), dtype=cache_dtype, device=dev)
    dec_algo_bytes = rec + d * cache.element_size()
    err = torch.full((2,), -1, dtype=torch.int64, device=dev)
    enc_layout = pool.kv_tensor_layout(shape, A, T)
    dec_layout = pool.kv_tensor_layout(shape, A, T, token_capacity=w["cache_tokens"],
                                       first_token=w["n_shared"])
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    stream = torch.cuda.current_stream().cuda_stream

    def step(ev=None):
        if ev:
            ev[0].record()
        prof.encode_dev(kv.data_ptr(), enc_layout, payload.data_ptr(), pstride, err.data_ptr(), stream)
        if ev:
            ev[1].record()
        prof.decode_patch_dev(payload.data_ptr(), pstride, dec_layout, cache.data_ptr(),
                              err[1:].data_ptr(), stream, dst_dtype=dst)
        if ev:
            ev[2].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        if not big:
            flush.zero_()
        step()
    torch.cuda.synchronize()
    assert int(err[0]) == -1 and int(err[1]) == -1, "a kernel reported a vector error"

    events = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = L.lib().pkv_launch_count()
    barrier()
    with ClockSampler(local) as clocks:
        t_wall = time.perf_counter()
        for i in range(args.steps):
            if not big:
                flush.zero_()  # evict the workload from L2; outside the per-step event bracket
            step(events[i])
        barrier()
        t_wall = time.perf_counter() - t_wall
    launches = L.lib().pkv_launch_count() - launches0
    enc_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in events]))
    dec_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in events]))
    step_ms = float(np.mean([e[0].elapsed_time(e[2]) for e in events]))

    # compressed-domain scoring of one query against the records just written (turbo only); outside
    # the timed region of the metric, reported beside it
    score = None
    if kind == "turbo":
        rq, pq = prof.prepare_query(np.random.default_rng(SEED).standard_normal(d).astype(np.float32))
        rq_dev = torch.from_numpy(rq).to(dev)
        pq_dev = torch.from_numpy(pq if pq.size else np.zeros(1, np.float32)).to(dev)
        scores = torch.empty(n_vec, dtype=torch.float32, device=dev)
        sev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(10)]
        for i in range(13):
            if not big:
                flush.zero_()
            if i >= 3:
                sev[i - 3][0].record()
            prof.score_dev(payload.data_ptr(), pstride, n_batches, vpb, rq_dev.data_ptr(), pq_dev.data_ptr(),
                           scores.data_ptr(), err[1:].data_ptr(), stream)
            if i >= 3:
                sev[i - 3][1].record()
        torch.cuda.synchronize()
        assert int(err[1]) == -1, "the score kernel reported a record"
        score_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in sev]))
        score = {"ms": score_ms, "records_per_s": n_vec / (score_ms * 1e-3),
                 "achieved_gbs": n_vec * (rec + 4) / (score_ms * 1e-3) / 1e9,
                 "api": "pkv_turbo_score_dev, one query against every record"}

    # end to end through the host-buffer C ABI: pinned host f32 -> TQB1 blobs -> pinned host f32
    blob = (L.FB2_HEADER_BYTES if kind == "fib" else L.TQB1_HEADER_BYTES) + vpb * rec
    x_host = torch.empty((n_batches, vpb, d), dtype=torch.float32).pin_memory()
    # gather order of the reference: token-major, head-minor per (agent, layer, side)
    x_host.copy_(kv.permute(0, 1, 2, 4, 3, 5).reshape(n_batches, vpb, d))
    wire_host = torch.empty((n_batches, blob), dtype=torch.uint8).pin_memory()
    out_host = torch.empty((n_batches, vpb, d), dtype=torch.float32).pin_memory()

    def e2e_step():
        pk.encode_batches_compact(prof, x_host.data_ptr(), n_batches, vpb, wire_host.data_ptr(),
                                  wire_host.numel())
        pk.decode_batches_compact(prof, wire_host.data_ptr(), n_batches, vpb, out_host.data_ptr(),
                                  out_host.numel())

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps

    times = torch.tensor([step_ms, enc_ms, dec_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    step_ms, enc_ms, dec_ms, e2e_ms = [float(v) for v in times.tolist()]

    if rank == 0:
        peak, peak_kind = measured_hbm_peak()
        total_f32 = 2 * f32_bytes * world
        value = total_f32 / (step_ms * 1e-3) / 1e9
        dom, dom_ms = (f"{kind}_encode_kernel<{d}>", enc_ms) if enc_ms >= dec_ms else (
            f"{kind}_decode_patch_kernel<{d}>", dec_ms)
        dom_bytes = algo_bytes if enc_ms >= dec_ms else dec_algo_bytes
        achieved = dom_bytes * n_vec / (dom_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["desc"], "vectors_per_gpu": n_vec, "f32_bytes_per_gpu": f32_bytes,
                       "parallelism": f"{world} x independent agent shards, no collective on the codec path",
                       "cache_dtype": args.cache_dtype,
                       "l2": "inputs larger than L2" if big else "flushed between timed steps (512 MiB write)"},
            "encode_gbs": f32_bytes * world / (enc_ms * 1e-3) / 1e9,
            "decode_patch_gbs": f32_bytes * world / (dec_ms * 1e-3) / 1e9,
            "encode_ms": enc_ms, "decode_patch_ms": dec_ms,
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": dom_bytes * n_vec,
                         "encode_achieved": algo_bytes * n_vec / (enc_ms * 1e-3) / 1e9,
                         "decode_patch_achieved": dec_algo_bytes * n_vec / (dec_ms * 1e-3) / 1e9,
                         "traffic": ncu_traffic(f"{args.workload}:{dom}")},
            "e2e": {"value": total_f32 / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (f32_bytes + n_batches * vpb * rec) * world,
                    "d2h_bytes_per_step": (f32_bytes + n_batches * vpb * rec) * world,
                    "api": f"pkv_{kind}_{{encode,decode}}_batches_compact, pinned host buffers"},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "wall_ms_timed_region": t_wall * 1e3,
        }
        if score is not None:
            score["frac_of_peak"] = score["achieved_gbs"] / peak
            line["score"] = score
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            gbs, t, sample = cpu_codec_rate(w, 8.0, cores)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--cache-dtype", default="f32", choices=["f32", "f16", "bf16"],
                    help="element type of the cache decode-and-patch writes (the metric counts f32 KV bytes "
                         "either way; the decode roofline counts the bytes actually written)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
