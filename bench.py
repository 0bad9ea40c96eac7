#!/usr/bin/env python
"""Benchmark of the bf16 GEMM hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

N = 1:  one step = one M=N=K=8192 bf16 GEMM (row-major A and B, f32 accumulate, f32 output, default
        auto_select config) -- the shape the headline metric is quoted on.  Inputs are synthetic
        N(0,1)/sqrt(K) bf16, created once and resident in HBM; A + B + C = 512 MiB > the 126 MB L2, so no
        explicit L2 flush is needed between iterations.
N > 1:  one step = the M=N=32768, K=8192 GEMM with bf16 output, B sharded by N-column blocks over the N GPUs,
        A replicated, every rank's full C filled by peer stores from the GEMM epilogue (strong scaling).

`value` is whole-job TFLOP/s (2*M*N*K per step / max-over-ranks device time).  `e2e` is the same metric
through the public C-ABI calls with HOST buffers: pinned host -> device copies of the operands and the
device -> host copy of the result inside the timed region.

`--impl reference` times the reference's CPU path for this GEMM (the C restatement of its host-side f32
reference matmul; the reference itself is Rust and cannot be built here) on all host threads, each step a
bounded row-slice of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "bf16 GEMM TFLOP/s"
UNIT = "TFLOP/s"
DENSE_PEAK_TFLOPS = 2250.0          # nominal B200 dense bf16
FALLBACK_PEAK_TFLOPS = 1590.0       # earlier measurement on this pool, used when MEASURED_PEAKS.json is absent


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_PEAK_TFLOPS, 1400.0, "fallback"


# ------------------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
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

    def _once(self):
        nv = self.nv
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                     "hw_power_brake_slowdown": 0x80, "sync_boost": 0x10, "applications_clocks_setting": 0x2}
            for k, bit in names.items():
                if r & bit:
                    self.reasons.add(k)
        except Exception:
            pass

    def _loop(self):
        while not self._stop.is_set():
            self._once()
            self._stop.wait(self.period)

    def start(self):
        if self.nv is None:
            return
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._once()
        self._stop.set()
        if self._thread:
            self._thread.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p for p in vis.split(",") if p.strip() != ""]
        try:
            return int(parts[local])
        except Exception:
            return local
    return local


# ------------------------------------------------------------------------------------------------ CPU side

def cpu_gemm_sample(m, n, k, seed_a, seed_b, target_s, threads):
    """Time the oracle's bf16 GEMM (k-ascending, unfused f32 mul+add) on a bounded row slice."""
    import numpy as np
    import oracle

    a_rows_max = min(m, 4096)
    scale = 1.0 / (k ** 0.5)
    b = oracle.normal_bf16((k, n), seed_b, scale)          # [K, N] row-major ("NN")
    a = oracle.normal_bf16((a_rows_max, k), seed_a, scale)
    probe = max(threads, 8)
    t0 = time.perf_counter()
    oracle.gemm_bf16(a, b, probe, n, k, trans_a=False, trans_b=False, threads=threads, row_end=probe)
    dt = time.perf_counter() - t0
    rows = int(max(probe, min(a_rows_max, probe * target_s / max(dt, 1e-6))))
    rows -= rows % max(threads, 1) if rows >= 2 * threads else 0
    return a, b, rows


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path, all host threads, bounded sample per step."""
    if rank != 0:
        return
    import oracle

    threads = os.cpu_count() or 1
    if world == 1:
        m, n, k, workload = 8192, 8192, 8192, "square_8192_nn_f32out"
    else:
        m, n, k, workload = 32768, 32768, 8192, f"colshard_32768x32768x8192_bf16out_g{world}"
    a, b, rows = cpu_gemm_sample(m, n, k, 1234, 1235, 1.5, threads)
    for _ in range(min(args.warmup, 1)):
        oracle.gemm_bf16(a, b, rows, n, k, trans_a=False, trans_b=False, threads=threads, row_end=rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.gemm_bf16(a, b, rows, n, k, trans_a=False, trans_b=False, threads=threads, row_end=rows)
    dt = (time.perf_counter() - t0) / args.steps
    val = 2.0 * rows * n * k / dt / 1e12
    sample = f"{rows} of {m} output rows x {n} cols, K={k}, per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "M": m, "N": n, "K": k, "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU side

def device_normal_bf16(torch, shape, seed, scale, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * scale).to(torch.bfloat16)


def time_steps(torch, fn, steps, stream):
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def context_measurements(torch, rt, L, stream, dev):
    """The memory-bound kernels (achieved HBM GB/s on working sets larger than L2) and the MLP training step of the
    fifth benchmark config at its per-GPU size (1024 rows), next to the headline GEMM number."""
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    out = {}
    hbm_peak = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            hbm_peak = float(json.load(f)["hbm_gbs"])
    except Exception:
        pass

    def gbs(fn, nbytes, steps=20):
        for _ in range(3):
            fn()
        ms = time_steps(torch, fn, steps, stream)
        g = nbytes / ms / 1e6
        return {"ms": ms, "gbs": g, "frac_of_measured_hbm": (g / hbm_peak) if hbm_peak else None}

    rows, cols = 8192, 4096
    nbuf = 4                                   # 4 x (128 MiB in + 128 MiB out): rotating so nothing is served from L2
    xs = [torch.randn(rows, cols, device=dev) for _ in range(nbuf)]
    ys = [torch.empty(rows, cols, device=dev) for _ in range(nbuf)]
    w = torch.ones(cols, device=dev)
    i = [0]

    def rms():
        j = i[0] % nbuf
        i[0] += 1
        rt._check(L.t0b_rmsnorm_fwd(rt.handle, xs[j].data_ptr(), w.data_ptr(), ys[j].data_ptr(), 0, rows, cols, 1e-6, 1))

    out["rmsnorm_fwd_8192x4096"] = gbs(rms, 2 * rows * cols * 4)
    dy = torch.randn(rows, cols, device=dev)

    def rms_bwd():
        j = i[0] % nbuf
        i[0] += 1
        rt._check(L.t0b_rmsnorm_bwd(rt.handle, dy.data_ptr(), xs[j].data_ptr(), w.data_ptr(), ys[j].data_ptr(), 0, 0, 0,
                                    rows, cols, 1e-6, 1))

    out["rmsnorm_bwd_dx_8192x4096"] = gbs(rms_bwd, 3 * rows * cols * 4)
    h16 = [torch.empty(rows, cols, device=dev, dtype=torch.bfloat16) for _ in range(nbuf)]
    dg = torch.empty(cols, device=dev)
    sb = L.t0b_rmsnorm_bwd_scratch_bytes(rows, cols)
    scratch = torch.empty(sb, dtype=torch.uint8, device=dev)

    def fused_fwd():
        j = i[0] % nbuf
        i[0] += 1
        rt._check(L.t0b_rmsnorm_silu_fwd(rt.handle, xs[j].data_ptr(), w.data_ptr(), h16[j].data_ptr(), 0, rows, cols, 1e-6, 1))

    def fused_bwd():
        j = i[0] % nbuf
        i[0] += 1
        rt._check(L.t0b_rmsnorm_silu_bwd(rt.handle, dy.data_ptr(), xs[j].data_ptr(), w.data_ptr(), h16[j].data_ptr(), dg.data_ptr(),
                                         scratch.data_ptr(), sb, rows, cols, 1e-6, 1))

    # algorithmic bytes: read x (f32) + write bf16; backward reads dh and x (f32), writes bf16 dx
    out["rmsnorm_silu_bf16_fwd_8192x4096"] = gbs(fused_fwd, rows * cols * 6)
    out["rmsnorm_silu_bf16_bwd_8192x4096"] = gbs(fused_bwd, rows * cols * 10)
    del xs, ys, dy, h16
    vocab, edim, tokens = 32000, 4096, 16384
    table = torch.randn(vocab, edim, device=dev)
    ids = torch.randint(0, vocab, (tokens,), device=dev, dtype=torch.int32)
    eout = torch.empty(tokens, edim, device=dev)
    gtab = torch.zeros(vocab, edim, device=dev)
    out["embedding_fwd_16384x4096"] = gbs(lambda: rt._check(L.t0b_embedding_fwd(
        rt.handle, table.data_ptr(), ids.data_ptr(), eout.data_ptr(), tokens, edim, vocab, 1)), 2 * tokens * edim * 4)
    uniq = int(torch.unique(ids).numel())
    out["embedding_bwd_16384x4096"] = gbs(lambda: rt._check(L.t0b_embedding_bwd(
        rt.handle, gtab.data_ptr(), ids.data_ptr(), eout.data_ptr(), tokens, edim, vocab, 0, 0, 1)),
        (tokens + 2 * uniq) * edim * 4)
    del table, eout, gtab
    rows, cols = 1024, 32000
    nbuf = 4
    xs = [torch.randn(rows, cols, device=dev) * 3 for _ in range(nbuf)]
    ds = [torch.empty(rows, cols, device=dev) for _ in range(nbuf)]
    tg = torch.randint(0, cols, (rows,), device=dev, dtype=torch.int32)
    loss = torch.empty(rows, device=dev)

    def ce():
        j = i[0] % nbuf
        i[0] += 1
        rt._check(L.t0b_softmax_ce(rt.handle, xs[j].data_ptr(), tg.data_ptr(), loss.data_ptr(), ds[j].data_ptr(), rows, cols,
                                   cols, 1.0 / rows, 1))

    out["softmax_ce_1024x32000"] = gbs(ce, 2 * rows * cols * 4)
    del xs, ds
    cfg = MlpConfig()
    tr = MlpTrainer(rt, cfg, 1024)
    x = torch.randn((1024, cfg.d_in), device=dev)
    t_ = torch.randint(0, cfg.n_classes, (1024,), device=dev, dtype=torch.int32)
    for _ in range(3):
        tr.step(x, t_)
    ms_fb = time_steps(torch, lambda: tr.forward_backward(x, t_), 10, stream)
    ms_step = time_steps(torch, lambda: tr.step(x, t_), 10, stream)
    out["mlp_step_1024rows_4096x3_32000"] = {"fwd_bwd_ms": ms_fb, "step_with_adamw_ms": ms_step,
                                             "gemm_tflops_fwd_bwd": cfg.flops_per_row() * 1024 / ms_fb / 1e9}
    return out


def run_single(args, local_rank):
    import torch

    import t0_gpu_b200 as t
    from t0_gpu_b200._lib import lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    rt = t.GpuRuntime(local_rank)
    # A dedicated (non-default) torch stream carries both the library's launches and the timing events.
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    rt.set_stream(stream.cuda_stream)
    L = lib()

    m = n = k = 8192
    a = device_normal_bf16(torch, (m, k), 1234, 1.0 / k ** 0.5, dev)
    b = device_normal_bf16(torch, (k, n), 1235, 1.0 / k ** 0.5, dev)       # [K, N] row-major
    c = torch.empty((m, n), dtype=torch.float32, device=dev)
    cfg = t.auto_select(m, k, n)

    def gemm(aa, bb, cc, mm, nn, kk, out_dtype=t.OUT_F32, async_=1):
        rt._check(L.t0b_gemm(rt.handle, None, 0, 0, aa.data_ptr(), bb.data_ptr(), cc.data_ptr(), mm, nn, kk, kk, nn, nn,
                             out_dtype, 0, 0, 1.0, 0, 0, async_))

    step = lambda: gemm(a, b, c, m, n, k)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    launches0 = rt.launch_count()
    sampler.start()
    ms = time_steps(torch, step, args.steps, stream)
    clocks = sampler.stop()
    launches = rt.launch_count() - launches0
    rt.synchronize()
    flops = 2.0 * m * n * k
    value = flops / (ms * 1e-3) / 1e12

    # Quick sanity of the timed output (the parity suite is tests/): a few rows against a f64 product.
    rows = [0, 4097, 8191]
    ref = (a[rows].double() @ b.double()).float()
    err = (c[rows] - ref).abs().max().item()
    if not err < 2 ** -7 * k ** 0.5 * 0.01:
        raise SystemExit(f"bench output failed its sanity check: max err {err}")

    # The other sizes of the sweep and the 1-GPU time of the sharded workload, for context.
    also = {}
    for s in (2048, 4096):
        aa, bb, cc = a[:s, :s].contiguous(), b[:s, :s].contiguous(), torch.empty((s, s), dtype=torch.float32, device=dev)
        f = lambda: gemm(aa, bb, cc, s, s, s)
        for _ in range(3):
            f()
        t_ms = time_steps(torch, f, max(args.steps, 20), stream)
        also[f"square_{s}_nn_f32out"] = {"ms": t_ms, "tflops": 2.0 * s ** 3 / (t_ms * 1e-3) / 1e12}
    # 256^3 is launch-bound: time it as a stream of launches and as one CUDA graph of 64 launches replayed.
    import ctypes as C
    s = 256
    aa, bb = a[:s, :s].contiguous(), b[:s, :s].contiguous()
    ccs = [torch.empty((s, s), dtype=torch.float32, device=dev) for _ in range(64)]
    f = lambda: gemm(aa, bb, ccs[0], s, s, s)
    for _ in range(3):
        f()
    t_stream = time_steps(torch, f, 200, stream)
    rt._check(L.t0b_graph_begin(rt.handle))
    for cc in ccs:
        gemm(aa, bb, cc, s, s, s)
    gh = C.c_uint64()
    rt._check(L.t0b_graph_end(rt.handle, C.byref(gh)))
    replay = lambda: rt._check(L.t0b_graph_launch(rt.handle, gh.value, 1))
    for _ in range(3):
        replay()
    t_graph = time_steps(torch, replay, 20, stream) / len(ccs)
    rt._check(L.t0b_graph_destroy(rt.handle, gh.value))
    also["square_256_nn_f32out"] = {"us_per_gemm_stream": t_stream * 1e3, "us_per_gemm_graph_of_64": t_graph * 1e3,
                                    "tflops_graph": 2.0 * s ** 3 / (t_graph * 1e-3) / 1e12}
    del ccs
    if not args.quick:
        bm, bn, bk = 32768, 32768, 8192
        a4 = device_normal_bf16(torch, (bm, bk), 4321, 1.0 / bk ** 0.5, dev)
        b4 = device_normal_bf16(torch, (bk, bn), 4322, 1.0 / bk ** 0.5, dev)
        c4 = torch.empty((bm, bn), dtype=torch.bfloat16, device=dev)
        f = lambda: gemm(a4, b4, c4, bm, bn, bk, out_dtype=t.OUT_BF16)
        for _ in range(2):
            f()
        t_ms = time_steps(torch, f, 5, stream)
        also["colshard_32768x32768x8192_bf16out_g1"] = {"ms": t_ms, "tflops": 2.0 * bm * bn * bk / (t_ms * 1e-3) / 1e12}
        del a4, b4, c4

    if not args.quick:
        also.update(context_measurements(torch, rt, L, stream, dev))

    # End to end through the C ABI with host buffers.
    a_h = a.cpu().pin_memory()
    b_h = b.cpu().pin_memory()
    c_h = torch.empty((m, n), dtype=torch.float32).pin_memory()

    def e2e_step():
        # The host-buffer entry point: copies of B, then row blocks of A, the GEMM of each block and the copy-back of
        # its block of C are pipelined on three streams inside the call.
        rt._check(L.t0b_gemm_host(rt.handle, None, 0, 0, a_h.data_ptr(), b_h.data_ptr(), c_h.data_ptr(), m, n, k, k, n, n,
                                  t.OUT_F32, 0))

    for _ in range(2):
        e2e_step()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = time_steps(torch, e2e_step, e2e_steps, stream)
    e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": (a_h.numel() + b_h.numel()) * 2,
           "d2h_bytes_per_step": c_h.numel() * 4, "ms_per_step": e2e_ms, "steps": e2e_steps,
           "api": "t0b_gemm_host (pinned host A, B, C; uploads, GEMM strips and read-back pipelined on three streams)"}
    if not torch.equal(c_h[4097].to(dev), c[4097]):
        raise SystemExit("bench: the host-buffer GEMM result differs from the device-resident one")

    burst, sustained, kind = measured_peak()
    long_region = ms * args.steps > 1000.0
    peak = sustained if long_region else burst
    roofline = {"bound": "tensor", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the
                # ncu capture summarised in profiles/gemm_bf16_tcgen05_8192cubed.md (algorithmic bytes: 536.9e6).
                "traffic": 1.1116e9, "peak_kind": f"of {kind} ({'sustained' if long_region else 'burst'} cuBLAS bf16)",
                "kernel": "gemm_bf16_tcgen05_kernel (tile " + cfg.name() + ")", "flops_per_launch": flops,
                "frac_of_nominal_dense_peak": value / DENSE_PEAK_TFLOPS}

    cpu = None
    if not args.no_cpu:
        import oracle
        threads = os.cpu_count() or 1
        a_s, b_s, rows_s = cpu_gemm_sample(m, n, k, 1234, 1235, 12.0, threads)
        t0 = time.perf_counter()
        oracle.gemm_bf16(a_s, b_s, rows_s, n, k, trans_a=False, trans_b=False, threads=threads, row_end=rows_s)
        dt = time.perf_counter() - t0
        cpu = {"value": 2.0 * rows_s * n * k / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{rows_s} of {m} output rows x {n} cols, K={k} ({dt:.1f} s)"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "square_8192_nn_f32out", "M": m, "N": n, "K": k, "gemm_config": cfg.name(),
                   "l2": "inputs+output 512 MiB > 126 MB L2, no flush", "accumulate": "f32", "output": "f32"},
        "pct_of_dense_peak": 100.0 * value / DENSE_PEAK_TFLOPS,
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
        "also": also,
    }
    print(json.dumps(line), flush=True)
    rt.close()


def run_multi(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    import t0_gpu_b200 as t
    from t0_gpu_b200._lib import lib
    from t0_gpu_b200.sharded import ColumnShardedGemm

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    rt = t.GpuRuntime(local_rank)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    rt.set_stream(stream.cuda_stream)
    L = lib()

    m, n, k = 32768, 32768, 8192
    op = ColumnShardedGemm(rt, m, n, k, out_dtype=t.OUT_BF16)
    sh = op.shard
    a = device_normal_bf16(torch, (m, k), 4321, 1.0 / k ** 0.5, dev)                  # replicated (same seed)
    b_full_cols = device_normal_bf16(torch, (k, n), 4322, 1.0 / k ** 0.5, dev)
    b = b_full_cols[:, sh.col0:sh.col0 + sh.n_local].contiguous()                      # this rank's column block
    del b_full_cols
    torch.cuda.empty_cache()

    class Buf:   # minimal GpuBuffer look-alike over torch memory
        def __init__(self, tensor):
            self.t = tensor

        def gpu_addr(self):
            return self.t.data_ptr()

    A, B = Buf(a), Buf(b)
    barrier = lambda: dist.barrier()

    def timed(fn, steps):
        barrier()
        torch.cuda.synchronize()
        ms = time_steps(torch, fn, steps, stream)
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        barrier()
        return tms.item()

    full = lambda: op.run(A, B, async_=True, gather=True)
    local = lambda: op.run(A, B, async_=True, gather=False)
    for _ in range(max(args.warmup, 3)):
        full()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    launches0 = rt.launch_count()
    sampler.start()
    ms = timed(full, args.steps)
    clocks = sampler.stop()
    launches = rt.launch_count() - launches0
    ms_local = timed(local, max(3, min(args.steps, 10)))
    rt.synchronize()
    flops = 2.0 * m * n * k
    value = flops / (ms * 1e-3) / 1e12

    # Every rank must now hold the same full C: compare a checksum of sampled rows across ranks, and a few
    # elements against an f64 product on rank 0.
    full()
    barrier()
    torch.cuda.synchronize()
    barrier()
    elem = 2
    rows = [0, 12345, m - 1]
    sample = torch.empty((len(rows), n), dtype=torch.bfloat16, device=dev)
    row_h = torch.empty(n, dtype=torch.bfloat16).pin_memory()
    for i, r in enumerate(rows):
        rt._check(L.t0b_memcpy_d2h(rt.handle, row_h.data_ptr(), op.c.gpu_addr() + r * n * elem, n * elem))
        sample[i] = row_h.to(dev)
    gathered = [torch.zeros_like(sample) for _ in range(world)]
    dist.all_gather(gathered, sample)
    same = all(torch.equal(gathered[0], g) for g in gathered)
    # each rank checks its own column block of the sampled rows against an f64 product of its operands
    ref = (a[rows].double() @ b.double()).to(torch.float32)
    got = sample[:, sh.col0:sh.col0 + sh.n_local].float()
    err = (got - ref).abs().max().item() if sh.n_local else 0.0
    ok = bool(same) and err < 0.02
    okt = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if okt.item() != 1:
        raise SystemExit(f"rank {rank}: sharded GEMM output failed its check (same={same}, err={err})")

    # End to end with host buffers: operands host -> device, this rank's output block device -> host.
    a_h = a.cpu().pin_memory()
    b_h = b.cpu().pin_memory()
    c_h = torch.empty((m, sh.n_local), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        rt._check(L.t0b_memcpy_h2d(rt.handle, a.data_ptr(), a_h.data_ptr(), a_h.numel() * 2))
        rt._check(L.t0b_memcpy_h2d(rt.handle, b.data_ptr(), b_h.data_ptr(), b_h.numel() * 2))
        op.run(A, B, async_=False, gather=True)
        rt._check(L.t0b_memcpy2d_d2h(rt.handle, c_h.data_ptr(), sh.n_local * elem, op.c.gpu_addr() + sh.col0 * elem,
                                     n * elem, sh.n_local * elem, m))

    e2e_step()
    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = timed(e2e_step, e2e_steps)
    e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": (a_h.numel() + b_h.numel()) * 2, "d2h_bytes_per_step": c_h.numel() * 2,
           "ms_per_step": e2e_ms, "steps": e2e_steps, "note": "bytes are per rank"}

    if rank == 0:
        burst, sustained, kind = measured_peak()
        per_gpu = value / world
        egress = (world - 1) * m * sh.n_local * elem
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"colshard_32768x32768x8192_bf16out_g{world}", "M": m, "N": n, "K": k,
                       "parallelism": f"B column-sharded x{world}, A replicated, all-gather fused into the GEMM epilogue (peer stores)",
                       "l2": "operands 0.5 GiB + output 2 GiB per GPU > L2, no flush", "output": "bf16"},
            "pct_of_dense_peak": 100.0 * per_gpu / DENSE_PEAK_TFLOPS,
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": sustained, "unit": UNIT,
                         "frac": per_gpu / sustained, "traffic": None,
                         "peak_kind": f"of {kind} (sustained cuBLAS bf16), per GPU",
                         "nvlink_egress_bytes_per_gpu": egress,
                         "nvlink_bound_ms": egress / 770e9 * 1e3,
                         "compute_bound_ms": flops / world / (sustained * 1e12) * 1e3,
                         "frac_of_fused_bound": max(egress / 770e9 * 1e3, flops / world / (sustained * 1e12) * 1e3) / ms},
            "gemm_only": {"ms_per_step": ms_local, "tflops": flops / (ms_local * 1e-3) / 1e12},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    op.close()
    barrier()
    dist.destroy_process_group()


def run_mlp(args, rank, local_rank, world):
    """--workload mlp: the data-parallel MLP training step of the fifth benchmark config (1024 rows per GPU,
    4096 -> 3 x [Linear 4096, RMSNorm, SiLU] -> Linear 32000 -> cross-entropy, AdamW), weak scaling over the ranks.
    A step = forward, backward, gradient exchange and optimizer update.  Inputs are resident; the value counts the
    GEMM FLOPs of forward and backward over all ranks."""
    import torch
    import torch.distributed as dist

    import t0_gpu_b200 as t
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rt = t.GpuRuntime(local_rank)
    cfg = MlpConfig()
    rows = 1024
    tr = MlpTrainer(rt, cfg, rows, rows_total=rows * world, shard_optimizer=not args.replicated_optimizer)
    g = torch.Generator(device=dev)
    g.manual_seed(7 + rank)
    x = torch.randn((rows, cfg.d_in), generator=g, device=dev)
    tg = torch.randint(0, cfg.n_classes, (rows,), generator=g, device=dev, dtype=torch.int32)

    def timed(fn, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = time_steps(torch, fn, steps, tr.stream)
        if world > 1:
            tms = torch.tensor([ms], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = tms.item()
        return ms

    step = lambda: tr.step(x, tg)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    launches0 = rt.launch_count()
    sampler.start()
    ms = timed(step, args.steps)
    clocks = sampler.stop()
    launches = rt.launch_count() - launches0
    ms_fb = timed(lambda: tr.forward_backward(x, tg), max(3, min(args.steps, 10)))
    loss = tr.mean_loss()
    flops = cfg.flops_per_row() * rows * world
    if rank == 0:
        print(json.dumps({
            "metric": "MLP training step, GEMM TFLOP/s (forward + backward FLOPs / step time)", "value": flops / (ms * 1e-3) / 1e12,
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlp_step_4096x3_32000_rows1024_per_gpu", "rows_per_gpu": rows, "global_batch": rows * world,
                       "optimizer": "AdamW, " + ("sharded over the ranks (reduce-scatter, all-gather)" if tr.sharded else
                                                 ("replicated (all-reduce)" if world > 1 else "single rank")),
                       "l2": "weights 363 MB bf16 + 726 MB f32 master per step > L2, no flush"},
            "fwd_bwd_ms": ms_fb, "loss": loss, "clocks": clocks, "gpu_launches": launches,
        }))
    if world > 1:
        dist.destroy_process_group()
    rt.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--quick", action="store_true", help="skip the 32768^2 single-GPU context measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload", default="gemm", choices=["gemm", "mlp"],
                    help="gemm: the headline GEMM (default); mlp: the data-parallel MLP training step")
    ap.add_argument("--replicated-optimizer", action="store_true",
                    help="--workload mlp on several GPUs: all-reduce + replicated AdamW instead of the sharded optimizer")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, max(world, args.gpus if world > 1 else 1))
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.workload == "mlp":
        run_mlp(args, rank, local_rank, world)
    elif world > 1:
        run_multi(args, rank, local_rank, world)
    else:
        run_single(args, local_rank)


if __name__ == "__main__":
    main()
