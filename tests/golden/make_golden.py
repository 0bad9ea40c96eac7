"""Collect the reference's golden vectors for the bf16 GEMM path into tests/golden/torch_ref/.

The reference ships a torch-generated fixture (benchmarks/torch_ref/, produced by its
benchmarks/gen_torch_ref.py and consumed by src/t0/precision_vs_torch.rs:302-305): bf16 inputs and
the f32 results of X*W^T for a SwiGLU block with M=64, K=256, N=512, seed 42.  This script copies
the files the oracle is pinned against, byte for byte, and records their SHA-256 so a later run can
tell whether the fixture changed.  Run it where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference
"""
import hashlib
import json
import os
import shutil
import sys

FILES = [
    "meta.txt",
    "x.bin",                 # bf16 [64, 256]
    "w_gate.bin",            # bf16 [512, 256]
    "w_up.bin",              # bf16 [512, 256]
    "w_down.bin",            # bf16 [256, 512]
    "h_gate_f32ref.bin",     # f32 [64, 512] = X * W_gate^T in f32
    "h_up_f32ref.bin",       # f32 [64, 512] = X * W_up^T in f32
    "swiglu_bf16_trunc.bin", # bf16 [64, 512] (truncated SwiGLU of the f32 refs)
    "y_bf16_f32acc.bin",     # f32 [64, 256] = swiglu_bf16_trunc * W_down^T in f32
]


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = sys.argv[1]
    src_dir = os.path.join(ref, "benchmarks", "torch_ref")
    dst_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "torch_ref")
    os.makedirs(dst_dir, exist_ok=True)
    sums = {}
    for name in FILES:
        src = os.path.join(src_dir, name)
        dst = os.path.join(dst_dir, name)
        shutil.copyfile(src, dst)
        with open(dst, "rb") as f:
            sums[name] = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(dst_dir, "SHA256.json"), "w") as f:
        json.dump(sums, f, indent=1, sort_keys=True)
    print(json.dumps(sums, indent=1, sort_keys=True))


if __name__ == "__main__":
    main()
