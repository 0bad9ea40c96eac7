"""Build the CPU oracle (oracle/t0_oracle.c) into oracle/_build/libt0_oracle.so.

Test infrastructure only: the oracle is the checker the CUDA library is compared against and the
timed CPU baseline; nothing in the product path links or calls it.

The reference project is Rust with no C/C++ sources, so there is nothing to compile from the
reference itself (no ``oracle/_ref`` build): the oracle is a C restatement pinned by the
reference's golden vectors (see tests/golden/).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "t0_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libt0_oracle.so")

# -ffp-contract=off: the reference accumulates with a separate f32 multiply and add.
CFLAGS = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-fvisibility=hidden", "-shared", "-fPIC", "-pthread"]


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", *CFLAGS, SRC, "-o", OUT, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
