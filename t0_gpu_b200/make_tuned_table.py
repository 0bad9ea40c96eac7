"""Measure the GEMM tile candidates on a B200 for the benchmark shapes (and the backward shapes of the MLP config)
and write the table that ships inside the library, csrc/t0b_tuned_table.inc.

    python -m t0_gpu_b200.make_tuned_table [--out PATH]

Needs a B200; every row is the winner of t0b_tune (all tiles x split-K x raster order, random operands) for one
shape, layout and output type.  After regenerating the table rebuild the library (python -m t0_gpu_b200.build).
It stands where the reference keeps its persistent tune cache (src/t0/cost_model.rs:788-1078, ~/.t0_autotune).
"""
from __future__ import annotations

import argparse
import os

from .gpu_context import OUT_BF16, OUT_F32, GpuRuntime

HERE = os.path.dirname(os.path.abspath(__file__))

PRESETS = {(256, 512): "b200_256x512", (512, 256): "b200_512x256", (256, 256): "b200_256x256", (256, 128): "b200_256x128",
           (128, 256): "b200_128x256", (128, 128): "b200_128x128", (128, 64): "b200_128x64"}


def shapes():
    """(M, N, K, trans_a, trans_b, out_dtype) of every benchmark config."""
    out = []
    for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):                       # config 1: 256^3 in every layout
        out.append((256, 256, 256, ta, tb, OUT_F32))
    for s in (512, 1024, 2048, 4096, 8192):                               # config 2: square sweep, row-major operands (512 and 1024: the reference's README table)
        out.append((s, s, s, 0, 0, OUT_F32))
        out.append((s, s, s, 0, 1, OUT_F32))
    for m, k, n in ((128, 4096, 4096), (4096, 4096, 128), (512, 16384, 512)):   # config 3: skinny and deep-K
        out.append((m, n, k, 0, 1, OUT_F32))
        out.append((m, n, k, 0, 0, OUT_F32))
    for g in (1, 2, 4, 8):                                                # config 4: per-GPU block of the sharded GEMM
        out.append((32768, 32768 // g, 8192, 0, 0, OUT_BF16))
    rows, d, v = 1024, 4096, 32000                                        # config 5: MLP step, 1024 rows per GPU
    out += [(rows, d, d, 0, 0, OUT_F32), (d, d, rows, 1, 0, OUT_F32), (rows, d, d, 0, 1, OUT_F32),      # hidden: fwd, dW, dX
            (rows, v, d, 0, 0, OUT_F32), (d, v, rows, 1, 0, OUT_F32), (d // 4, v, rows, 1, 0, OUT_F32),  # output: fwd, dW (whole, panel)
            (rows, d, v, 0, 1, OUT_F32)]                                                                # output: dX
    seen, uniq = set(), []
    for s in out:
        if s not in seen:
            seen.add(s)
            uniq.append(s)
    return uniq


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "csrc", "t0b_tuned_table.inc"))
    args = ap.parse_args()
    rt = GpuRuntime(0)
    lines = ["// Shipped autotune table.  Generated on a B200 by `python -m t0_gpu_b200.make_tuned_table` (t0b_tune over the",
             "// benchmark shapes and their backward shapes); one row per shape, layout and output type:",
             "//   {M, N, K, trans_a, trans_b, out_bf16, tile preset, split_k, swap_grid, raster group, measured TFLOP/s}"]
    for (m, n, k, ta, tb, od) in shapes():
        cfg, tf = rt.tune(m, n, k, trans_a=bool(ta), trans_b=bool(tb), out_dtype=od)
        preset = PRESETS[(cfg.tile_m, cfg.tile_n)]
        lines.append('{%d, %d, %d, %d, %d, %d, "%s", %d, %d, %d, %.1ff},' % (m, n, k, ta, tb, int(od == OUT_BF16), preset, cfg.split_k or 0,
                                                                           int(cfg.swap_grid), cfg.lds_pad, tf))
        print(lines[-1], flush=True)
    lines.append('{0, 0, 0, 0, 0, 0, "b200_128x128", 0, 0, 0, 0.0f},   // terminator (never matches: shapes are non-zero)')
    with open(args.out, "w") as f:
        f.write("\n".join(lines) + "\n")
    rt.close()
    print("wrote", args.out)


if __name__ == "__main__":
    main()
