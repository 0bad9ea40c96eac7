"""Host-side mirror of the reference's GEMM autotuner (src/t0/auto_gemm.rs): `GemmTuner` (measure, cache in memory
and on disk in the reference's JSON wire format), `global_tuner()`, and the one-shot `auto_gemm`.  Measuring is done
by the C ABI's on-device tuner (t0b_tune); this module only keeps the reference's bookkeeping around it."""
from __future__ import annotations

import ctypes as C
import os
import shutil
import sys
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ._lib import GemmConfigC, lib
from .gemm_gen import GemmConfig


def default_cache_dir() -> str:
    """$T0_AUTOTUNE_DIR, else ~/.t0_autotune (src/t0/auto_gemm.rs:484-492)."""
    return os.environ.get("T0_AUTOTUNE_DIR") or os.path.join(os.environ.get("HOME", "."), ".t0_autotune")


@dataclass
class GemmTuneResult:
    """struct GemmTuneResult (src/t0/auto_gemm.rs:29-41)."""
    best: GemmConfig
    best_tflops: float
    all: List[Tuple[str, float]]
    key: Tuple[int, int, int]
    from_cache: bool


@dataclass
class GemmTuner:
    """struct GemmTuner (src/t0/auto_gemm.rs:46-78).  `max_candidates` and `n_iters` are kept for source
    compatibility; the device tuner measures its whole (small) candidate list with five timed launches each."""
    cache_dir: str = field(default_factory=default_cache_dir)
    max_candidates: int = 8
    n_iters: int = 5
    cache: Dict[Tuple[int, int, int], GemmTuneResult] = field(default_factory=dict)

    @staticmethod
    def new() -> "GemmTuner":
        return GemmTuner()

    @staticmethod
    def with_cache_dir(directory: str) -> "GemmTuner":
        return GemmTuner(cache_dir=str(directory))

    def cache_path(self, m: int, n: int, k: int) -> str:
        return os.path.join(self.cache_dir, f"gemm_{m}x{n}x{k}.json")

    def load_cache(self, m: int, n: int, k: int) -> Optional[GemmTuneResult]:
        cfg, tf = GemmConfigC(), C.c_float()
        if lib().t0b_tune_cache_load(self.cache_dir.encode(), m, n, k, C.byref(cfg), C.byref(tf)) != 0:
            return None
        return GemmTuneResult(GemmConfig.from_c(cfg), float(tf.value), [], (m, n, k), True)

    def tune(self, rt, m: int, n: int, k: int) -> GemmConfig:
        """GemmTuner::tune(rt, m, n, k) (src/t0/auto_gemm.rs:82-162), argument order (M, N, K): memory cache, then
        the disk cache, then a measurement on the device whose result is written to both."""
        key = (m, n, k)
        hit = self.cache.get(key)
        if hit is not None:
            return hit.best
        cached = self.load_cache(m, n, k)
        if cached is not None:
            print(f"[autotune] Cache hit: {m}x{n}x{k} -> {cached.best.name()} ({cached.best_tflops:.1f} TFLOPS)", file=sys.stderr)
            self.cache[key] = cached
            # make config-less GEMM calls of this shape use the cached choice as well
            rt._check(lib().t0b_set_autotune_dir(rt.handle, self.cache_dir.encode()))
            rt.tune(m, n, k)
            return cached.best
        rt._check(lib().t0b_set_autotune_dir(rt.handle, self.cache_dir.encode()))
        best, tflops = rt.tune(m, n, k)                      # measures, fills the runtime's table, writes the JSON file
        print(f"[autotune] Best: {best.name()} ({tflops:.1f} TFLOPS)", file=sys.stderr)
        self.cache[key] = GemmTuneResult(best, tflops, [(best.name(), tflops)], key, False)
        return best

    def invalidate(self, m: int, n: int, k: int) -> None:
        """auto_gemm.rs:394-397."""
        self.cache.pop((m, n, k), None)
        lib().t0b_tune_cache_invalidate(self.cache_dir.encode(), m, n, k)

    def clear(self) -> None:
        """auto_gemm.rs:400-403: forget everything, remove the cache directory."""
        self.cache.clear()
        shutil.rmtree(self.cache_dir, ignore_errors=True)

    def report(self, file=None) -> None:
        """auto_gemm.rs:406-417."""
        file = file or sys.stderr
        print(f"GEMM Autotune Cache ({len(self.cache)} entries)", file=file)
        for (m, n, k), r in self.cache.items():
            print(f"  {m}x{n}x{k} -> {r.best.name()} ({r.best_tflops:.1f} TF) {'[cached]' if r.from_cache else '[measured]'}", file=file)


_GLOBAL: Optional[GemmTuner] = None
_GLOBAL_LOCK = threading.Lock()


def global_tuner() -> GemmTuner:
    """The lazily created process-wide tuner (src/t0/auto_gemm.rs:425-431)."""
    global _GLOBAL
    with _GLOBAL_LOCK:
        if _GLOBAL is None:
            _GLOBAL = GemmTuner.new()
        return _GLOBAL


def auto_gemm(rt, a_buf, b_buf, c_buf, m: int, n: int, k: int) -> float:
    """auto_gemm(rt, a, b, c, m, n, k) (src/t0/auto_gemm.rs:445-480): tune (or hit the cache), run
    C[M,N] f32 = A[M,K] bf16 x B[N,K]^T bf16 with the best config, return the TFLOP/s the tuner measured.
    The reference goes through the 40-byte kernarg blob, which needs tile-aligned M and N; the direct call used here
    takes any shape."""
    tuner = global_tuner()
    cfg = tuner.tune(rt, m, n, k)
    rt.gemm(a_buf, b_buf, c_buf, m, n, k, cfg=cfg, trans_a=False, trans_b=True)
    r = tuner.cache.get((m, n, k))
    return r.best_tflops if r else 0.0
