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
bounded row-slice of the same workload, in the reference's own NT form (both operands K-contiguous, B transposed
once on the host outside the timed region as Ignis does).
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
FALLBACK_PEAK_TFLOPS = 1590.0       # cuBLAS bf16 burst on a B200, used when MEASURED_PEAKS.json is absent
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the GEMM kernel on the 8192^3 workload, from an ncu
# capture of `python bench.py --quick --no-cpu --steps 2 --warmup 1`, keyed by the tile the run chose (algorithmic
# bytes: 536.9e6).  A tile without a capture reports traffic null.
NCU_DRAM_TRAFFIC_8192 = {
    "t0_gemm_256x512_k64_ldsdb_wgp": 1.1116e9,
}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_PEAK_TFLOPS, 1400.0, "fallback"


def measured_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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

def cpu_gemm_sample(m, n, k, seed_a, seed_b, target_s, threads, layout="NT"):
    """Operands and a row count for timing the oracle's bf16 GEMM (k-ascending, unfused f32 mul+add) on a bounded row
    slice.  layout "NT": B stored [N, K] like the reference's own CPU loop (examples/test_gemm_correctness.rs:28-42;
    Ignis transposes W once on the host first, src/ignis/ops/bf16_matmul.rs:390-424) -- the transpose is done here,
    outside every timed region.  layout "NN": B stored [K, N], read with a stride of N (the layout the GPU arm is given)."""
    import numpy as np
    import oracle

    a_rows_max = min(m, 4096)
    scale = 1.0 / (k ** 0.5)
    b = oracle.normal_bf16((k, n), seed_b, scale)          # [K, N] row-major
    if layout == "NT":
        b = np.ascontiguousarray(b.T)                      # [N, K]
    a = oracle.normal_bf16((a_rows_max, k), seed_a, scale)
    tb = layout == "NT"
    probe = max(threads, 8)
    t0 = time.perf_counter()
    oracle.gemm_bf16(a, b, probe, n, k, trans_a=False, trans_b=tb, threads=threads, row_end=probe)
    dt = time.perf_counter() - t0
    rows = int(max(probe, min(a_rows_max, probe * target_s / max(dt, 1e-6))))
    rows -= rows % max(threads, 1) if rows >= 2 * threads else 0
    return a, b, rows


def cpu_gemm_time(a, b, rows, n, k, threads, layout):
    import oracle

    t0 = time.perf_counter()
    oracle.gemm_bf16(a, b, rows, n, k, trans_a=False, trans_b=(layout == "NT"), threads=threads, row_end=rows)
    return time.perf_counter() - t0


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path, all host threads, bounded sample per step."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    if world == 1:
        m, n, k, workload = 8192, 8192, 8192, "square_8192_nn_f32out"
    else:
        m, n, k, workload = 32768, 32768, 8192, f"colshard_32768x32768x8192_bf16out_g{world}"
    a, b, rows = cpu_gemm_sample(m, n, k, 1234, 1235, 1.5, threads, "NT")
    for _ in range(min(args.warmup, 1)):
        cpu_gemm_time(a, b, rows, n, k, threads, "NT")
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_gemm_time(a, b, rows, n, k, threads, "NT")
    dt = (time.perf_counter() - t0) / args.steps
    val = 2.0 * rows * n * k / dt / 1e12
    sample = f"{rows} of {m} output rows x {n} cols, K={k}, per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "M": m, "N": n, "K": k, "sample": sample,
                   "layout": "NT (B stored [N, K], transposed once on the host outside the timed region)"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample, "layout": "NT"},
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


def row_kernel_measurements(torch, rt, L, stream, dev, norm_sizes=((8192, 4096),), ce_sizes=((1024, 32000),), embedding=True):
    """The memory-bound kernels: achieved HBM GB/s over their algorithmic bytes.  Every operand is rotated through four
    buffer sets (more than 0.5 GiB per kernel) so that nothing is served from the 126 MB L2; each figure is the median
    of five timings of 20 back-to-back launches after three warm-ups, CUDA events on the launching stream."""
    out = {}
    hbm_peak, hbm_kind = measured_hbm()

    def gbs(fn, nbytes, steps=20):
        for _ in range(3):
            fn()
        ms = statistics.median(time_steps(torch, fn, steps, stream) for _ in range(5))
        g = nbytes / ms / 1e6
        return {"ms": ms, "gbs": g, "frac_of_measured_hbm": g / hbm_peak, "hbm_peak_kind": hbm_kind, "algorithmic_bytes": nbytes}

    nbuf = 4
    i = [0]

    def nxt():
        j = i[0] % nbuf
        i[0] += 1
        return j

    for rows, cols in norm_sizes:
        tag = f"{rows}x{cols}"
        xs = [torch.randn(rows, cols, device=dev) for _ in range(nbuf)]
        ys = [torch.empty(rows, cols, device=dev) for _ in range(nbuf)]
        dys = [torch.randn(rows, cols, device=dev) for _ in range(nbuf)]
        h16 = [torch.empty(rows, cols, device=dev, dtype=torch.bfloat16) for _ in range(nbuf)]
        w = torch.ones(cols, device=dev)
        dg = torch.empty(cols, device=dev)
        sb = L.t0b_rmsnorm_bwd_scratch_bytes(rows, cols)
        scratch = torch.empty(sb, dtype=torch.uint8, device=dev)

        def rms():
            j = nxt()
            rt._check(L.t0b_rmsnorm_fwd(rt.handle, xs[j].data_ptr(), w.data_ptr(), ys[j].data_ptr(), 0, rows, cols, 1e-6, 1))

        def rms_bwd_dx():
            j = nxt()
            rt._check(L.t0b_rmsnorm_bwd(rt.handle, dys[j].data_ptr(), xs[j].data_ptr(), w.data_ptr(), ys[j].data_ptr(), 0, 0, 0,
                                        rows, cols, 1e-6, 1))

        def rms_bwd():
            j = nxt()
            rt._check(L.t0b_rmsnorm_bwd(rt.handle, dys[j].data_ptr(), xs[j].data_ptr(), w.data_ptr(), ys[j].data_ptr(), dg.data_ptr(),
                                        scratch.data_ptr(), sb, rows, cols, 1e-6, 1))

        def fused_fwd():
            j = nxt()
            rt._check(L.t0b_rmsnorm_silu_fwd(rt.handle, xs[j].data_ptr(), w.data_ptr(), h16[j].data_ptr(), 0, rows, cols, 1e-6, 1))

        def fused_bwd():
            j = nxt()
            rt._check(L.t0b_rmsnorm_silu_bwd(rt.handle, dys[j].data_ptr(), xs[j].data_ptr(), w.data_ptr(), h16[j].data_ptr(),
                                             dg.data_ptr(), scratch.data_ptr(), sb, rows, cols, 1e-6, 1))

        out[f"rmsnorm_fwd_{tag}"] = gbs(rms, 2 * rows * cols * 4)
        out[f"rmsnorm_bwd_dx_{tag}"] = gbs(rms_bwd_dx, 3 * rows * cols * 4)
        out[f"rmsnorm_bwd_dx_dgamma_{tag}"] = gbs(rms_bwd, 3 * rows * cols * 4)
        # algorithmic bytes: read x (f32) + write bf16; backward reads dh and x (f32), writes bf16 dx
        out[f"rmsnorm_silu_bf16_fwd_{tag}"] = gbs(fused_fwd, rows * cols * 6)
        out[f"rmsnorm_silu_bf16_bwd_{tag}"] = gbs(fused_bwd, rows * cols * 10)
        del xs, ys, dys, h16
    if embedding:
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
    for rows, cols in ce_sizes:
        xs = [torch.randn(rows, cols, device=dev) * 3 for _ in range(nbuf)]
        ds = [torch.empty(rows, cols, device=dev) for _ in range(nbuf)]
        d16 = [torch.empty(rows, cols, device=dev, dtype=torch.bfloat16) for _ in range(nbuf)]
        tg = torch.randint(0, cols, (rows,), device=dev, dtype=torch.int32)
        loss = torch.empty(rows, device=dev)

        def ce():
            j = nxt()
            rt._check(L.t0b_softmax_ce(rt.handle, xs[j].data_ptr(), tg.data_ptr(), loss.data_ptr(), ds[j].data_ptr(), rows, cols,
                                       cols, 1.0 / rows, 1))

        def ce16():
            j = nxt()
            rt._check(L.t0b_softmax_ce_bf16(rt.handle, xs[j].data_ptr(), tg.data_ptr(), loss.data_ptr(), d16[j].data_ptr(), rows, cols,
                                            cols, 1.0 / rows, 1))

        out[f"softmax_ce_{rows}x{cols}"] = gbs(ce, 2 * rows * cols * 4)
        out[f"softmax_ce_bf16grad_{rows}x{cols}"] = gbs(ce16, rows * cols * 6)
        del xs, ds, d16
    return out


def context_measurements(torch, rt, L, stream, dev):
    """The MLP training step of the fifth benchmark config at its per-GPU size (1024 rows), next to the headline GEMM."""
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    out = {}
    cfg = MlpConfig()
    tr = MlpTrainer(rt, cfg, 1024, autotune=False)   # the shapes of this step are in the shipped table
    x = torch.randn((1024, cfg.d_in), device=dev)
    t_ = torch.randint(0, cfg.n_classes, (1024,), device=dev, dtype=torch.int32)
    for _ in range(3):
        tr.step(x, t_)
    ms_fb = time_steps(torch, lambda: tr.forward_backward(x, t_), 10, stream)
    ms_step = time_steps(torch, lambda: tr.step(x, t_), 10, stream)
    out["mlp_step_1024rows_4096x3_32000"] = {"fwd_bwd_ms": ms_fb, "step_with_adamw_ms": ms_step,
                                             "gemm_tflops_fwd_bwd": cfg.flops_per_row() * 1024 / ms_fb / 1e9}
    return out


def run_skinny(args, local_rank):
    """--workload skinny: only the skinny / split-K GEMMs of the third benchmark config (one GPU)."""
    import torch

    import t0_gpu_b200 as t
    from t0_gpu_b200._lib import lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    rt = t.GpuRuntime(local_rank)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    rt.set_stream(stream.cuda_stream)
    res = skinny_splitk_measurements(torch, t, rt, lib(), stream, dev)
    hbm, kind = measured_hbm()
    print(json.dumps({"metric": "skinny and split-K bf16 GEMMs, microseconds per call (GEMM + reduce)", "unit": "us", "n_gpus": 1,
                      "hbm_peak": hbm, "peak_kind": f"of {kind} copy bandwidth", "shapes": res,
                      "config": {"workload": "skinny_splitk", "l2": "eight operand sets rotated (280 MiB) > L2"}}), flush=True)
    rt.close()


def run_timeline(args, local_rank):
    """--workload timeline: where a GEMM launch spends its time, from %globaltimer stamps inside the kernels.  Uses the
    timeline build of the library (libt0b200_trace.so: the same sources with -DT0B_TRACE, `python -m
    t0_gpu_b200.build --trace`), its own context, and t0b_trace_set.  Sixteen launches go out back to back; the last
    four are reported, each phase as the median over the CTAs of the launch."""
    import ctypes as C

    import numpy as np
    import torch

    from t0_gpu_b200._lib import load_trace_lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    L = load_trace_lib()
    ctx = C.c_void_p()
    if L.t0b_ctx_create(local_rank, C.byref(ctx)) != 0:
        raise SystemExit("t0b_ctx_create failed in the timeline build")
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    assert L.t0b_ctx_set_stream(ctx, stream.cuda_stream) == 0
    slots, ctas = 8, 160
    trace = torch.zeros(slots * ctas * 16, dtype=torch.int64, device=dev)
    shapes = [(256, 256, 256), (128, 4096, 4096), (2048, 2048, 2048), (1024, 4096, 4096), (4096, 4096, 4096)]
    out = {}
    for (m, n, k) in shapes:
        a = device_normal_bf16(torch, (m, k), 77, 1.0 / k ** 0.5, dev)
        b = device_normal_bf16(torch, (k, n), 78, 1.0 / k ** 0.5, dev)
        cs = [torch.empty((m, n), dtype=torch.float32, device=dev) for _ in range(4)]
        torch.cuda.synchronize()

        def launch(i):
            rc = L.t0b_gemm(ctx, None, 0, 0, a.data_ptr(), b.data_ptr(), cs[i & 3].data_ptr(), m, n, k, k, n, n, 0, 0, 0, 1.0, 0, 0, 1)
            if rc != 0:
                raise SystemExit(f"t0b_gemm failed: {rc}")

        for i in range(4):
            launch(i)
        assert L.t0b_sync(ctx) == 0
        trace.zero_()
        torch.cuda.synchronize()
        assert L.t0b_trace_set(ctx, trace.data_ptr(), slots) == 0
        for i in range(2 * slots):
            launch(i)
        assert L.t0b_sync(ctx) == 0
        assert L.t0b_trace_set(ctx, 0, 0) == 0
        tr = trace.cpu().numpy().reshape(slots, ctas, 16)      # launches 8..15, in order
        rows = []
        for li in range(slots - 4, slots):
            cur, prev = tr[li], tr[li - 1]
            live = cur[:, 0] > 0
            med = lambda slot: float(np.median(cur[live & (cur[:, slot] > 0), slot])) if (live & (cur[:, slot] > 0)).any() else None
            prev_end = float(prev[prev[:, 14] > 0, 14].max())
            prev_dep = float(np.median(prev[prev[:, 2] > 0, 2]))
            dep, issue, data, mma, acc, staged, stored = med(2), med(3), med(4), med(5), med(6), med(7), med(8)
            end = float(cur[live, 14].max())
            # Slots 12 / 13 hold %globaltimer values (close to the other stamps) in a cluster split-K launch, cycle counters otherwise.
            csk = med(13) is not None and bool((np.abs(cur[live, 13] - cur[live, 0]) < 1_000_000_000).all())
            ph = {"previous_launch_gone_to_dependency_wait_done": dep - prev_end, "to_first_k_block_issued": issue - dep,
                  "to_first_operands_in_smem": data - issue, "main_loop": mma - data, "to_accumulator_complete": acc - mma}
            if csk:
                ph["accumulator_to_shared_memory"] = staged - acc
                ph["cluster_barrier"] = med(13) - staged
                ph["sum_over_dsmem_and_closing_barrier"] = med(12) - med(13)
                ph["teardown"] = end - med(12)
            else:
                ph["epilogue_stores_complete"] = stored - acc
                ph["teardown"] = end - stored
                mm = live & (cur[:, 12] > 0) & (cur[:, 13] > cur[:, 12])
                if mm.any():
                    ghz = (cur[mm, 13] - cur[mm, 12]).astype(float) / (cur[mm, 5] - cur[mm, 4]).astype(float)
                    ph["sm_clock_ghz_main_loop"] = float(np.median(ghz))
            ph = {kk: (round(v / 1000.0, 2) if not kk.startswith("sm_clock") else round(v, 3)) for kk, v in ph.items()}
            ph["period"] = round((dep - prev_dep) / 1000.0, 2)
            rows.append(ph)
        keys = rows[0].keys()
        out[f"{m}x{n}x{k}_nn_f32out"] = {"ctas": int((tr[slots - 1][:, 0] > 0).sum()), "cluster_split_k": bool(csk),
                                          "us_median_of_last_4_launches": {kk: round(float(np.median([r[kk] for r in rows])), 3) for kk in keys}}
        del a, b, cs
    L.t0b_ctx_destroy(ctx)
    print(json.dumps({"metric": "GEMM launch timeline from in-kernel %globaltimer stamps (timeline build), microseconds",
                      "unit": "us", "n_gpus": 1, "shapes": out,
                      "config": {"workload": "timeline", "launches": "16 back to back, programmatic dependent launch; the last 4 reported",
                                 "library": "libt0b200_trace.so (-DT0B_TRACE)"}}), flush=True)


def run_rows(args, local_rank):
    """--workload rows: only the memory-bound kernels, at the sizes of the table in profiles/ (one GPU)."""
    import torch

    import t0_gpu_b200 as t
    from t0_gpu_b200._lib import lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    rt = t.GpuRuntime(local_rank)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    rt.set_stream(stream.cuda_stream)
    sampler = ClockSampler(physical_gpu_index(local_rank), period_s=0.02)
    sampler.start()
    if args.quick:     # the small set a profiler capture uses (about 2 GiB resident at a time)
        res = row_kernel_measurements(torch, rt, lib(), stream, dev, embedding=False)
    else:
        res = row_kernel_measurements(torch, rt, lib(), stream, dev, norm_sizes=((1024, 4096), (8192, 4096), (32768, 4096)),
                                      ce_sizes=((1024, 32000), (8192, 32000)))
    clocks = sampler.stop()
    hbm, kind = measured_hbm()
    print(json.dumps({"metric": "memory-bound kernels, achieved HBM GB/s over algorithmic bytes", "unit": "GB/s", "n_gpus": 1,
                      "peak": hbm, "peak_kind": f"of {kind} copy bandwidth", "clocks": clocks, "kernels": res,
                      "config": {"workload": "row_kernels", "l2": "operands rotated through four buffer sets > L2"}}), flush=True)
    rt.close()


def skinny_splitk_measurements(torch, t, rt, L, stream, dev):
    """The third benchmark config: skinny GEMMs and the deep-K GEMM with split_k 4 and 8 (uniform[-1,1) bf16 inputs in
    the reference's NT layout, f32 output).  One timed call = everything t0b_gemm launches for the shape -- with
    split-K that is the GEMM AND the fixed-order reduce.  These shapes are HBM-bound (35 / 35 / 33 MiB of operands and
    output per call), so each also reports GB/s over its algorithmic bytes 2(MK + KN) + 4MN against the measured
    copy bandwidth; eight operand sets are rotated so that consecutive calls do not find their data in L2."""
    hbm_peak, hbm_kind = measured_hbm()
    out = {}
    nset = 8
    cases = [("skinny_m128_k4096_n4096", 128, 4096, 4096, 0), ("skinny_m4096_k4096_n128", 4096, 4096, 128, 0),
             ("splitk4_m512_k16384_n512", 512, 16384, 512, 4), ("splitk8_m512_k16384_n512", 512, 16384, 512, 8)]
    for name, m, k, n, sk in cases:
        g = torch.Generator(device=dev)
        g.manual_seed(m * 1000 + k)
        xs = [(torch.rand((m, k), generator=g, device=dev) * 2 - 1).to(torch.bfloat16) for _ in range(nset)]
        ws = [(torch.rand((n, k), generator=g, device=dev) * 2 - 1).to(torch.bfloat16) for _ in range(nset)]
        ys = [torch.empty((m, n), dtype=torch.float32, device=dev) for _ in range(nset)]
        i = [0]
        cc = [None]

        def call():
            j = i[0] % nset
            i[0] += 1
            rt._check(L.t0b_gemm(rt.handle, C.byref(cc[0]), 0, 1, xs[j].data_ptr(), ws[j].data_ptr(), ys[j].data_ptr(), m, n, k,
                                 k, k, n, t.OUT_F32, 0, 0, 1.0, 0, 0, 1))

        cfg = t.auto_select(m, k, n)
        if sk:
            # split_k is pinned by the benchmark config; the tile is the one that runs fastest WITH that split (a short
            # timing of every B200 tile preset, as the tuner does when split_k is free).
            best = None
            for name_ in ("b200_128x64", "b200_128x128", "b200_128x256", "b200_256x128", "b200_256x256"):
                cand = t.GemmConfig.preset(name_).with_(split_k=sk)
                cc[0] = cand.to_c()
                for _ in range(nset):
                    call()
                ms_c = time_steps(torch, call, 24, stream)
                if best is None or ms_c < best[0]:
                    best = (ms_c, cand)
            cfg = best[1]
        cc[0] = cfg.to_c()
        for _ in range(nset):
            call()
        l0 = rt.launch_count()
        ms = statistics.median(time_steps(torch, call, 40, stream) for _ in range(5))
        launches_per_call = (rt.launch_count() - l0) / 200.0
        ref = xs[(i[0] - 1) % nset][:4].double() @ ws[(i[0] - 1) % nset].double().T
        err = (ys[(i[0] - 1) % nset][:4].double() - ref).abs().max().item()
        if not err < 2 ** -7 * k ** 0.5:
            raise SystemExit(f"bench: {name} failed its sanity check: max err {err}")
        nbytes = 2 * (m * k + k * n) + 4 * m * n
        gbs = nbytes / ms / 1e6
        out[name] = {"us": ms * 1e3, "tflops": 2.0 * m * n * k / (ms * 1e-3) / 1e12, "gbs": gbs,
                     "frac_of_hbm": gbs / hbm_peak, "hbm_peak_kind": hbm_kind, "algorithmic_bytes": nbytes,
                     "config": cfg.name(), "launches_per_call": launches_per_call,
                     "timed": "GEMM + split-K reduce together" if (cfg.split_k or 0) > 1 else "GEMM"}
        del xs, ws, ys
    return out


def sustained_measurement(torch, step, ms_estimate, flops, stream, gpu_index, seconds=2.5):
    """The headline GEMM back to back for `seconds` (power-capped clocks), with the SM clock sampled beside it."""
    n = max(50, int(seconds * 1e3 / ms_estimate))
    sampler = ClockSampler(gpu_index, period_s=0.02)
    sampler.start()
    ms = time_steps(torch, step, n, stream)
    clk = sampler.stop()
    burst, sustained, kind = measured_peak()
    tf = flops / (ms * 1e-3) / 1e12
    mhz = clk.get("sm_mhz")
    return {"launches": n, "seconds": ms * n / 1e3, "ms": ms, "tflops": tf, "frac_of_sustained_cublas": tf / sustained,
            "peak_kind": f"of {kind} (sustained cuBLAS bf16)", "sm_mhz_median": mhz,
            "ms_x_mhz": (ms * mhz) if mhz else None, "reasons": clk.get("reasons"), "power_w_max": clk.get("power_w_max")}


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

    # Order of the measurements.  The latency- and memory-bound kernels (row kernels, the skinny / split-K GEMMs) go first,
    # on a GPU that has not yet been loaded: after a run of large GEMMs at the power cap the SM clock stays near its
    # sustained value (about 1.3 GHz against 1.97) for a while, and these kernels then take 13 % (row kernels) to 50 %
    # (skinny GEMMs) longer until the GPU has idled for about a second (measured).  The square sweep follows in ascending
    # size (2048, 4096, then the headline 8192 with its own warm-up), then the long-running context measurements
    # (32768^2, the sustained loop, the MLP step).
    rows_first = {} if (args.quick or args.headline_only) else row_kernel_measurements(torch, rt, L, stream, dev)
    skinny_first = {} if args.headline_only else skinny_splitk_measurements(torch, t, rt, L, stream, dev)
    # The MLP step (config 5 at its per-GPU size) is measured here too, before the GPU has been loaded: after the sustained
    # loops below the same step reads 2.25 ms instead of 1.92 (measured, with a 1.5 s pause in between).
    mlp_first = {} if (args.quick or args.headline_only) else context_measurements(torch, rt, L, stream, dev)

    m = n = k = 8192
    a = device_normal_bf16(torch, (m, k), 1234, 1.0 / k ** 0.5, dev)
    b = device_normal_bf16(torch, (k, n), 1235, 1.0 / k ** 0.5, dev)       # [K, N] row-major
    c = torch.empty((m, n), dtype=torch.float32, device=dev)
    cfg = t.auto_select(m, k, n)

    def gemm(aa, bb, cc, mm, nn, kk, out_dtype=t.OUT_F32, async_=1):
        rt._check(L.t0b_gemm(rt.handle, None, 0, 0, aa.data_ptr(), bb.data_ptr(), cc.data_ptr(), mm, nn, kk, kk, nn, nn,
                             out_dtype, 0, 0, 1.0, 0, 0, async_))

    # The smaller squares of the sweep (sizes ascending, as the reference's sweep runs them), each a burst of a few
    # milliseconds on a GPU that is not yet at its power cap -- the state the burst peak they are compared with was
    # measured in; `sustained_8192` below is the seconds-long counterpart.
    also = {}
    squares_first = {}
    def measure_256():
        """256^3 is launch-bound: time it as a stream of launches and as one CUDA graph of 64 launches replayed."""
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
        return {"us_per_gemm_stream": t_stream * 1e3, "us_per_gemm_graph_of_64": t_graph * 1e3,
                "tflops_graph": 2.0 * s ** 3 / (t_graph * 1e-3) / 1e12}

    if not args.headline_only:
        squares_first["square_256_nn_f32out"] = measure_256()
    for s in (() if args.headline_only else (2048, 4096)):
        aa, bb, cc = a[:s, :s].contiguous(), b[:s, :s].contiguous(), torch.empty((s, s), dtype=torch.float32, device=dev)
        f = lambda: gemm(aa, bb, cc, s, s, s)
        for _ in range(3):
            f()
        t_ms = time_steps(torch, f, max(args.steps, 20), stream)
        squares_first[f"square_{s}_nn_f32out"] = {"ms": t_ms, "tflops": 2.0 * s ** 3 / (t_ms * 1e-3) / 1e12}
        del aa, bb, cc

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

    # Quick sanity of the timed output (the parity suite is tests/): a few rows against a f64 product, within the
    # GEMM tolerance 2^-7 * sqrt(K) * max|a| * max|b|.
    rows = [0, 4097, 8191]
    ref = (a[rows].double() @ b.double()).float()
    err = (c[rows] - ref).abs().max().item()
    bound = 2 ** -7 * k ** 0.5 * a.abs().max().item() * b.abs().max().item()
    if not err < bound:
        raise SystemExit(f"bench output failed its sanity check: max err {err} (bound {bound})")

    also.update(squares_first)
    if args.headline_only:
        # The short command of the profiler captures: the headline launches come first, then the launch-bound case.
        also["square_256_nn_f32out"] = measure_256()
        args.quick = True
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

    also.update(skinny_first)
    also.update(rows_first)
    if not args.quick:
        also["sustained_8192"] = sustained_measurement(torch, step, ms, flops, stream, physical_gpu_index(local_rank))
        # The same loop with bf16 output, the form of the cuBLAS run behind the sustained peak (torch.matmul of bf16
        # tensors writes bf16): like for like, half the C bytes.
        c16 = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        step16 = lambda: gemm(a, b, c16, m, n, k, out_dtype=t.OUT_BF16)
        for _ in range(3):
            step16()
        also["sustained_8192_bf16out"] = sustained_measurement(torch, step16, ms, flops, stream, physical_gpu_index(local_rank), seconds=1.5)
        del c16
        also.update(mlp_first)

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
    traffic = NCU_DRAM_TRAFFIC_8192.get(cfg.name())
    roofline = {"bound": "tensor", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak,
                "traffic": traffic, "traffic_note": ("ncu capture of this tile" if traffic else "no capture for this tile"),
                "algorithmic_bytes": 2.0 * (m * k + k * n) + 4.0 * m * n,
                "peak_kind": f"of {kind} ({'sustained' if long_region else 'burst'} cuBLAS bf16)",
                "kernel": "gemm_bf16_tcgen05_kernel (tile " + cfg.name() + ")", "flops_per_launch": flops,
                "frac_of_nominal_dense_peak": value / DENSE_PEAK_TFLOPS}

    cpu = None
    if not args.no_cpu:
        threads = os.cpu_count() or 1
        # The reference's own form first: NT, both operands K-contiguous.  Then, on a smaller sample, the NN form the
        # GPU arm is given (B read with a stride of N), to show how much of the difference is layout.
        a_s, b_s, rows_s = cpu_gemm_sample(m, n, k, 1234, 1235, 10.0, threads, "NT")
        dt = cpu_gemm_time(a_s, b_s, rows_s, n, k, threads, "NT")
        cpu = {"value": 2.0 * rows_s * n * k / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port", "layout": "NT",
               "sample": f"{rows_s} of {m} output rows x {n} cols, K={k} ({dt:.1f} s)"}
        a_s, b_s, rows_n = cpu_gemm_sample(m, n, k, 1234, 1235, 4.0, threads, "NN")
        dt = cpu_gemm_time(a_s, b_s, rows_n, n, k, threads, "NN")
        cpu["nn_layout"] = {"value": 2.0 * rows_n * n * k / dt / 1e12,
                            "sample": f"{rows_n} of {m} output rows x {n} cols, K={k} ({dt:.1f} s)"}
        del a_s, b_s

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


def mlp_measurement(torch, dist, rt, rank, world, dev, steps, warmup, replicated):
    """The data-parallel MLP training step of the fifth benchmark config at `world` ranks (1024 rows per GPU,
    4096 -> 3 x [Linear 4096, RMSNorm, SiLU] -> Linear 32000 -> cross-entropy, AdamW).  A step = forward, backward,
    gradient exchange and optimizer update; inputs are resident.  Returns rank-identical numbers (max over ranks)."""
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    cfg = MlpConfig()
    rows = 1024
    tr = MlpTrainer(rt, cfg, rows, rows_total=rows * world, shard_optimizer=not replicated)
    g = torch.Generator(device=dev)
    g.manual_seed(7 + rank)
    x = torch.randn((rows, cfg.d_in), generator=g, device=dev)
    tg = torch.randint(0, cfg.n_classes, (rows,), generator=g, device=dev, dtype=torch.int32)

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = time_steps(torch, fn, n, tr.stream)
        if world > 1:
            tms = torch.tensor([ms], device=dev)
            dist.all_reduce(tms, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = tms.item()
        return ms

    step = lambda: tr.step(x, tg)
    for _ in range(max(warmup, 3)):
        step()
    launches0 = rt.launch_count()
    ms = timed(step, steps)
    launches = rt.launch_count() - launches0
    ms_fb = timed(lambda: tr.forward_backward(x, tg), max(3, min(steps, 10)))
    loss = tr.mean_loss()
    tr.finish_updates()
    rt.synchronize()
    flops = cfg.flops_per_row() * rows * world
    out = {"ms_per_step": ms, "fwd_bwd_ms": ms_fb, "gemm_tflops_whole_job": flops / (ms * 1e-3) / 1e12, "loss": loss,
           "rows_per_gpu": rows, "global_batch": rows * world, "launches_per_step": launches / steps,
           "optimizer": "AdamW, " + ("sharded over the ranks (reduce-scatter, all-gather)" if tr.sharded else
                                     ("replicated (fp32 gradient all-reduce)" if world > 1 else "single rank"))}
    del tr, x, tg
    torch.cuda.empty_cache()
    return out


def dp_equivalence_check(torch, dist, rt, rank, world, dev):
    """`world` ranks, each with its slice of a 128-row batch of a reduced MLP (256-wide, 512 classes), must give the
    gradients and the loss of one rank that sees the whole batch: relative Frobenius error <= 1e-3 (the row-kernel
    tolerance; the sums are reassociated across ranks), loss to 1e-5."""
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    cfg = MlpConfig(d_in=256, hidden=[256, 256, 256], n_classes=512)
    rows_total = 128
    rows = rows_total // world
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    x = torch.randn((rows_total, 256), generator=g, device=dev)
    g.manual_seed(8)
    tg = torch.randint(0, 512, (rows_total,), generator=g, device=dev, dtype=torch.int32)
    tr = MlpTrainer(rt, cfg, rows, rows_total=rows_total, autotune=False)
    tr.forward_backward(x[rank * rows:(rank + 1) * rows].contiguous(), tg[rank * rows:(rank + 1) * rows].contiguous())
    rt.synchronize()
    loss_dp = tr.mean_loss()
    one = MlpTrainer(rt, cfg, rows_total, rows_total=rows_total, autotune=False, local_only=True)
    one.forward_backward(x, tg)
    rt.synchronize()
    loss_one = one.mean_loss()
    rel = ((tr.grads - one.grads).norm() / one.grads.norm()).item()
    ok = rel <= 1e-3 and abs(loss_dp - loss_one) <= 1e-5 * abs(loss_one) + 1e-6
    okt = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    return {"ranks_equal_one_rank": bool(okt.item() == 1), "grad_rel_frobenius": rel, "loss_dp": loss_dp, "loss_one_rank": loss_one,
            "shape": "128 rows, 256 -> 3 x 256 -> 512"}


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
    elem = 2
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

    # ---- checks on the WHOLE output, outside every timed region.
    # (1) every rank holds the same full C: block-wise checksums of all 2 GiB, computed on the device, compared across ranks.
    op.c.zero()
    barrier()
    full()
    op.finish()
    block = 1 << 20
    nblocks = (m * n * elem + block - 1) // block
    sums = torch.zeros(2 * nblocks, dtype=torch.int64, device=dev)
    rt._check(L.t0b_hash_blocks(rt.handle, op.c.gpu_addr(), m * n * elem, block, sums.data_ptr(), 0))
    gathered = [torch.zeros_like(sums) for _ in range(world)]
    dist.all_gather(gathered, sums)
    full_c_equal = all(torch.equal(gathered[0], g) for g in gathered)
    # (2) this rank's own column block equals, bit for bit, what a plain single-destination GEMM computes for it.
    own = torch.empty((m, sh.n_local), dtype=torch.bfloat16, device=dev)
    rt._check(L.t0b_gemm(rt.handle, None, 0, 0, a.data_ptr(), b.data_ptr(), own.data_ptr(), m, sh.n_local, k, k, sh.n_local,
                         sh.n_local, t.OUT_BF16, 0, 0, 1.0, 0, 0, 0))
    got = torch.empty_like(own)
    rt._check(L.t0b_copy_d2d(rt.handle, got.data_ptr(), sh.n_local * elem, op.c.gpu_addr() + sh.col0 * elem, n * elem,
                             sh.n_local * elem, m, 0))
    own_block_bit_identical = bool(torch.equal(own.view(torch.int16), got.view(torch.int16)))
    # (3) and a few rows of it against an f64 product, within the GEMM tolerance (+ bf16 output rounding).
    rows = [0, 12345, m - 1]
    ref = (a[rows].double() @ b.double()).to(torch.float32)
    err = (got[rows].float() - ref).abs().max().item()
    bound = 2 ** -7 * k ** 0.5 * a.abs().max().item() * b.abs().max().item() + 2 ** -8 * ref.abs().max().item()
    ok = full_c_equal and own_block_bit_identical and err < bound
    okt = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if okt.item() != 1:
        raise SystemExit(f"rank {rank}: sharded GEMM output failed its check (full_c_equal={full_c_equal}, "
                         f"own_block_bit_identical={own_block_bit_identical}, err={err}, bound={bound})")
    checks = {"full_c_equal": True, "own_block_bit_identical": True, "max_abs_err_vs_f64_rows": err,
              "how": f"{nblocks} block checksums of each rank's 2 GiB C compared across ranks; own column block "
                     "recomputed by a plain t0b_gemm and compared bit for bit"}
    del own, got, sums, gathered

    # ---- the NVLink store rate the fused all-gather is bounded by: this library's own copy kernel (SM-issued 16-byte
    # stores, like the epilogue's) writing this rank's column block into the next rank's C, all ranks at once.
    peer_gbs = None
    if world > 1 and sh.n_local:
        src = op.c.gpu_addr() + sh.col0 * elem
        dst = op._peer_ptrs[1] + sh.col0 * elem            # the same block in the peer's C: the bytes are already equal
        cp = lambda: rt._check(L.t0b_copy_d2d(rt.handle, dst, n * elem, src, n * elem, sh.n_local * elem, m, 1))
        cp()
        ms_cp = timed(cp, 3)
        peer_gbs = m * sh.n_local * elem / ms_cp / 1e6
        op.finish()

    # ---- end to end from pinned HOST buffers.  A is replicated, so every rank uploads only its 1/world row slice of A
    # (and its B shard) over PCIe and the slices are all-gathered over NVLink; the GEMM then runs in row strips and each
    # finished strip of this rank's output block travels to the host while the next strip is multiplied.
    a_rows = m // world
    a_h = a[rank * a_rows:(rank + 1) * a_rows].cpu().pin_memory()
    b_h = b.cpu().pin_memory()
    c_h = torch.empty((m, sh.n_local), dtype=torch.bfloat16).pin_memory()
    a_slice = a[rank * a_rows:(rank + 1) * a_rows]
    strips = 8
    srows = m // strips
    # This rank's column block leaves the device as dense rows: a strided read-back of 2/world-GiB in rows of
    # n_local * 2 bytes at a 64 KiB pitch reaches only ~34 GB/s over PCIe, a dense one ~57 GB/s.
    dense = torch.empty((m, sh.n_local), dtype=torch.bfloat16, device=dev)

    def e2e_step():
        rt._check(L.t0b_memcpy_h2d_async(rt.handle, a_slice.data_ptr(), a_h.data_ptr(), a_h.numel() * 2))
        rt._check(L.t0b_memcpy_h2d_async(rt.handle, b.data_ptr(), b_h.data_ptr(), b_h.numel() * 2))
        dist.all_gather_into_tensor(a, a_slice)                      # in place: slice r sits at rows [r*a_rows, ...)
        for i in range(strips):
            op.run(A, B, async_=True, gather=True, rows=(i * srows, srows))
            strip_bytes = srows * sh.n_local * elem
            rt._check(L.t0b_copy_d2d(rt.handle, dense.data_ptr() + i * strip_bytes, sh.n_local * elem,
                                     op.c.gpu_addr() + (i * srows * n + sh.col0) * elem, n * elem, sh.n_local * elem, srows, 1))
            rt._check(L.t0b_memcpy2d_d2h_async(rt.handle, c_h.data_ptr() + i * strip_bytes, sh.n_local * elem,
                                               dense.data_ptr() + i * strip_bytes, sh.n_local * elem, sh.n_local * elem, srows))
        rt.synchronize()

    e2e_step()
    barrier()
    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = timed(e2e_step, e2e_steps)
    if not torch.equal(c_h[12345].to(dev).view(torch.int16), ref_row_bits(torch, op, rt, L, sh, n, elem, 12345, dev)):
        raise SystemExit(f"rank {rank}: the host copy of C differs from the device copy")
    # each leg alone, once, for the record
    legs = {}
    legs["h2d_a_slice_b_shard"] = timed(lambda: (rt._check(L.t0b_memcpy_h2d_async(rt.handle, a_slice.data_ptr(), a_h.data_ptr(), a_h.numel() * 2)),
                                                 rt._check(L.t0b_memcpy_h2d_async(rt.handle, b.data_ptr(), b_h.data_ptr(), b_h.numel() * 2)),
                                                 rt.synchronize()), 2)
    legs["allgather_a_nvlink"] = timed(lambda: dist.all_gather_into_tensor(a, a_slice), 2)
    legs["gemm_fused_gather"] = ms
    legs["d2h_own_block_dense"] = timed(lambda: (rt._check(L.t0b_memcpy2d_d2h_async(rt.handle, c_h.data_ptr(), sh.n_local * elem,
                                                                                    dense.data_ptr(), sh.n_local * elem, sh.n_local * elem, m)),
                                                 rt.synchronize()), 2)
    e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": (a_h.numel() + b_h.numel()) * 2, "d2h_bytes_per_step": c_h.numel() * 2,
           "ms_per_step": e2e_ms, "steps": e2e_steps, "note": "bytes are per rank", "legs_alone_ms": legs,
           "api": "t0b_memcpy_h2d_async (1/world row slice of A + the B shard), NCCL all-gather of A over NVLink, "
                  f"t0b_gemm_multi_dst in {strips} row strips, t0b_copy_d2d of each strip of the own block into dense rows, "
                  "t0b_memcpy2d_d2h_async of each strip, t0b_sync"}
    op.close()
    del a, b, a_h, b_h, c_h, A, B, a_slice, dense, ref
    torch.cuda.empty_cache()

    # ---- the data-parallel MLP training step (fifth config) at the same ranks: the all-reduce form and the sharded optimizer.
    mlp = {"allreduce_replicated_adamw": mlp_measurement(torch, dist, rt, rank, world, dev, 10, 3, True),
           "sharded_optimizer": mlp_measurement(torch, dist, rt, rank, world, dev, 10, 3, False),
           "equivalence": dp_equivalence_check(torch, dist, rt, rank, world, dev)}
    if not mlp["equivalence"]["ranks_equal_one_rank"]:
        raise SystemExit(f"rank {rank}: the data-parallel gradients differ from the one-rank gradients: {mlp['equivalence']}")

    if rank == 0:
        burst, sustained, kind = measured_peak()
        per_gpu = value / world
        ingress = (world - 1) * m * sh.n_local * elem           # = egress: (G-1)/G * 2 GiB per GPU
        link_gbs = peer_gbs if peer_gbs else 713.0
        link_ms = ingress / (link_gbs * 1e9) * 1e3
        long_region = ms * args.steps > 1000.0          # the same rule as the one-GPU line: burst peak for a short timed region
        peak = sustained if long_region else burst
        compute_ms = flops / world / (peak * 1e12) * 1e3
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"colshard_32768x32768x8192_bf16out_g{world}", "M": m, "N": n, "K": k,
                       "parallelism": f"B column-sharded x{world}, A replicated, all-gather fused into the GEMM epilogue (peer stores)",
                       "gemm_config": t.sharded.multi_dst_config(m, k, sh.n_local, world, rt.num_sms()).name(),
                       "l2": "operands 0.5 GiB + output 2 GiB per GPU > L2, no flush", "output": "bf16"},
            "pct_of_dense_peak": 100.0 * per_gpu / DENSE_PEAK_TFLOPS,
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "checks": checks,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": UNIT,
                         "frac": per_gpu / peak, "traffic": None,
                         "peak_kind": f"of {kind} ({'sustained' if long_region else 'burst'} cuBLAS bf16), per GPU",
                         "nvlink_ingress_bytes_per_gpu": ingress,
                         "nvlink_store_gbs_measured": peer_gbs,
                         "nvlink_store_how": "t0b_copy_d2d of this rank's column block into the next rank's C, all ranks at once",
                         "nvlink_bound_ms": link_ms, "compute_bound_ms": compute_ms,
                         "frac_of_fused_bound": max(link_ms, compute_ms) / ms},
            "gemm_only": {"ms_per_step": ms_local, "tflops": flops / (ms_local * 1e-3) / 1e12},
            "cpu_baseline": None,
            "also": {"mlp_step": mlp},
        }
        print(json.dumps(line), flush=True)
    barrier()
    dist.destroy_process_group()
    rt.close()


def ref_row_bits(torch, op, rt, L, sh, n, elem, row, dev):
    """Row `row` of this rank's own column block, read from the device copy of C, as int16 bit patterns."""
    out = torch.empty(sh.n_local, dtype=torch.bfloat16, device=dev)
    rt._check(L.t0b_copy_d2d(rt.handle, out.data_ptr(), sh.n_local * elem, op.c.gpu_addr() + (row * n + sh.col0) * elem,
                             sh.n_local * elem, sh.n_local * elem, 1, 0))
    return out.view(torch.int16)


def run_mlp(args, rank, local_rank, world):
    """--workload mlp: the data-parallel MLP training step of the fifth benchmark config (1024 rows per GPU,
    4096 -> 3 x [Linear 4096, RMSNorm, SiLU] -> Linear 32000 -> cross-entropy, AdamW), weak scaling over the ranks.
    A step = forward, backward, gradient exchange and optimizer update.  Inputs are resident; the value counts the
    GEMM FLOPs of forward and backward over all ranks."""
    import torch
    import torch.distributed as dist

    import t0_gpu_b200 as t

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rt = t.GpuRuntime(local_rank)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    r = mlp_measurement(torch, dist, rt, rank, world, dev, args.steps, args.warmup, args.replicated_optimizer)
    clocks = sampler.stop()
    if rank == 0:
        print(json.dumps({
            "metric": "MLP training step, GEMM TFLOP/s (forward + backward FLOPs / step time)", "value": r["gemm_tflops_whole_job"],
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlp_step_4096x3_32000_rows1024_per_gpu", "rows_per_gpu": r["rows_per_gpu"],
                       "global_batch": r["global_batch"], "optimizer": r["optimizer"],
                       "l2": "weights 363 MB bf16 + 726 MB f32 master per step > L2, no flush"},
            "fwd_bwd_ms": r["fwd_bwd_ms"], "loss": r["loss"], "clocks": clocks,
            "gpu_launches": int(r["launches_per_step"] * args.steps),
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
    ap.add_argument("--headline-only", action="store_true",
                    help="time only the headline GEMM (plus 256^3 and the host-buffer leg): the short command profiler captures use")
    ap.add_argument("--workload", default="gemm", choices=["gemm", "mlp", "rows", "skinny", "timeline"],
                    help="gemm: the headline GEMM (default); mlp: the data-parallel MLP training step; "
                         "rows: the memory-bound row kernels alone (one GPU); skinny: the skinny / split-K GEMMs alone (one GPU); "
                         "timeline: phases of a GEMM launch from in-kernel timer stamps (needs the --trace build of the library)")
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
    if args.workload in ("rows", "skinny", "timeline"):
        if rank == 0:
            {"rows": run_rows, "skinny": run_skinny, "timeline": run_timeline}[args.workload](args, local_rank)
    elif args.workload == "mlp":
        run_mlp(args, rank, local_rank, world)
    elif world > 1:
        run_multi(args, rank, local_rank, world)
    else:
        run_single(args, local_rank)


if __name__ == "__main__":
    main()
