"""Build libt0b200.so (the C-ABI CUDA library) in-tree for sm_100a with nvcc.

    python -m t0_gpu_b200.build [--force] [--verbose] [--trace]

The library is cross-compiled (no GPU needed) and lands in t0_gpu_b200/lib/libt0b200.so; `--trace` builds the timeline
variant (the same sources with -DT0B_TRACE) as t0_gpu_b200/lib/libt0b200_trace.so.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OUT = os.path.join(OUT_DIR, "libt0b200.so")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
# The timeline build: the same sources with -DT0B_TRACE (the GEMM kernels stamp %globaltimer at their phase changes).
TRACE_OUT = os.path.join(OUT_DIR, "libt0b200_trace.so")
TRACE_OBJ_DIR = os.path.join(OUT_DIR, "obj_trace")

SOURCES = ["t0b_runtime.cu", "t0b_gemm.cu", "t0b_rowops.cu", "t0b_embedding.cu", "t0b_util.cu", "t0b_gemm_gen.cpp", "t0b_tile_ir.cpp"]
# The GEMM kernel variants (BN, CG, MT, ND): gemm_variant.cu compiled once per entry, side by side.
GEMM_VARIANTS = ["256,2,2,1", "256,2,2,0", "256,2,1,0", "128,2,1,0", "256,1,1,0", "128,1,1,0", "64,1,1,0"]
HEADERS = ["gemm_sm100.cuh", "gemm_launch.cuh", "ptx_sm100.cuh", "t0b_internal.hpp", "t0b_tuned_table.inc", os.path.join("..", "..", "include", "t0b200.h")]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    out, obj_dir = (TRACE_OUT, TRACE_OBJ_DIR) if trace else (OUT, OBJ_DIR)
    extra = ["-DT0B_TRACE"] if trace else []
    # Up to date already (e.g. a built library shipped without its object files): nothing to do.
    all_inputs = [os.path.join(CSRC, f) for f in SOURCES + HEADERS + ["gemm_variant.cu"]]
    if not force and os.path.exists(out) and os.path.getmtime(out) >= _newest(all_inputs):
        return out
    os.makedirs(obj_dir, exist_ok=True)
    hdr_time = _newest([os.path.join(CSRC, h) for h in HEADERS])
    objs, jobs = [], []
    units = [(src, os.path.splitext(src)[0] + ".o", []) for src in SOURCES]
    units += [("gemm_variant.cu", "gemm_variant_" + v.replace(",", "_") + ".o", ["-DT0B_V_%s=%s" % (k, x) for k, x in zip(("BN", "CG", "MT", "ND"), v.split(","))])
              for v in GEMM_VARIANTS]
    for src, obj_name, defines in units:
        sp = os.path.join(CSRC, src)
        obj = os.path.join(obj_dir, obj_name)
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(sp), hdr_time)
        if stale:
            cmd = [NVCC, *ARCH, *CFLAGS, *extra, *defines, "-c", sp, "-o", obj]
            if src.endswith(".cpp"):
                cmd.insert(1, "-x")
                cmd.insert(2, "cu")
            if verbose:
                cmd += ["-Xptxas", "-v"]
                print(" ".join(cmd), flush=True)
            jobs.append(cmd)
    # The translation units are independent: compile them side by side.
    procs = [subprocess.Popen(cmd) for cmd in jobs]
    failed = [cmd for cmd, p in zip(jobs, procs) if p.wait() != 0]
    if failed:
        raise subprocess.CalledProcessError(1, failed[0])
    if force or not os.path.exists(out) or os.path.getmtime(out) < _newest(objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", out, *objs, "-cudart", "static"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
