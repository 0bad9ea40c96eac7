"""Host-side mirror of the reference's GEMM generator API (src/t0/gemm_gen.rs, re-exported at
src/t0/mod.rs:61-67): same names, argument orders and error behaviour, each a thin call into the C ABI.

Argument orders follow the reference exactly, including its inconsistencies:
``auto_select(m, k, n)`` but ``build_kernargs(x, wt, y, k, n, m, cfg)``.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, replace
from typing import Optional

from ._lib import GemmConfigC, GemmPlanC, lib


class GemmTranspose(enum.IntEnum):
    NT = 0   # Y[M,N] = A[M,K] @ B[N,K]^T
    NN = 1   # Y[M,N] = A[M,K] @ B[K,N]


class EpilogueOp(enum.IntEnum):
    StoreF32 = 0
    BiasAddStoreF32 = 1
    BiasAddReluStoreF32 = 2
    # tile_ir single-op epilogues
    Relu = 3
    SiLU = 4
    GeluSigmoid = 5
    Scale = 6
    Abs = 7
    Neg = 8


@dataclass
class GemmConfig:
    """`struct GemmConfig`, src/t0/gemm_gen.rs:55-84 (public fields, clonable)."""
    tile_m: int
    tile_n: int
    tile_k: int
    wg_size: int
    use_lds: bool = True
    double_buffer: bool = True
    split_k: Optional[int] = None
    lds_pad: int = 0
    n_col_passes: int = 1
    swap_grid: bool = True
    wgp_mode: bool = True
    transpose: GemmTranspose = GemmTranspose.NT
    epilogue: EpilogueOp = EpilogueOp.StoreF32

    # ---- C struct round trip
    def to_c(self) -> GemmConfigC:
        return GemmConfigC(self.tile_m, self.tile_n, self.tile_k, self.wg_size, int(self.use_lds),
                           int(self.double_buffer), self.split_k or 0, self.lds_pad, self.n_col_passes,
                           int(self.swap_grid), int(self.wgp_mode), int(self.transpose), int(self.epilogue))

    @staticmethod
    def from_c(c: GemmConfigC) -> "GemmConfig":
        return GemmConfig(c.tile_m, c.tile_n, c.tile_k, c.wg_size, bool(c.use_lds), bool(c.double_buffer),
                          c.split_k or None, c.lds_pad, c.n_col_passes, bool(c.swap_grid), bool(c.wgp_mode),
                          GemmTranspose(c.transpose), EpilogueOp(c.epilogue))

    def with_(self, **kw) -> "GemmConfig":
        """Struct-update syntax (`GemmConfig { split_k: Some(4), ..preset }`)."""
        return replace(self, **kw)

    # ---- presets (gemm_gen.rs:86-145) and the B200-native tiles
    @staticmethod
    def preset(name: str) -> "GemmConfig":
        c = GemmConfigC()
        if lib().t0b_config_preset(name.encode(), C.byref(c)) != 0:
            raise ValueError(f"unknown GemmConfig preset {name!r}")
        return GemmConfig.from_c(c)

    # ---- derived getters (gemm_gen.rs:147-205)
    def n_col_tiles(self) -> int:
        return self.tile_n // 16

    def n_waves(self) -> int:
        return self.wg_size // 32

    def rows_per_wave(self) -> int:
        return self.tile_m // self.n_waves()

    def n_row_blocks(self) -> int:
        return self.rows_per_wave() // 16

    def k_sub_steps(self) -> int:
        return self.tile_k // 16

    def lds_per_buffer(self) -> int:
        return self.tile_m * self.tile_k * 2 + self.tile_n * self.tile_k * 2

    def lds_total(self) -> int:
        return lib().t0b_config_lds_total(C.byref(self.to_c()))

    def estimated_vgprs(self) -> int:
        return lib().t0b_config_estimated_vgprs(C.byref(self.to_c()))

    def is_feasible(self) -> bool:
        return bool(lib().t0b_config_is_feasible(C.byref(self.to_c())))

    def name(self) -> str:
        buf = C.create_string_buffer(160)
        n = lib().t0b_config_name(C.byref(self.to_c()), buf, 160)
        if n < 0:
            raise ValueError("t0b_config_name failed")
        return buf.value.decode()


for _p in ("16x64_k16", "32x64_direct", "32x64_k16", "32x64_k32", "32x128_k16", "64x64_k16", "64x64_k32",
           "128x64_k16", "64x128_k16", "128x64_k32", "128x128_k16", "64x64_k64", "128x128_2pass", "64x128_2pass"):
    setattr(GemmConfig, "tile_" + _p, staticmethod(lambda _n=_p: GemmConfig.preset(_n)))


def _list(fn) -> list:
    arr = (GemmConfigC * 32)()
    n = fn(arr, 32)
    return [GemmConfig.from_c(arr[i]) for i in range(n)]


def sweep_configs() -> list:
    return _list(lib().t0b_sweep_configs)


def standard_configs() -> list:
    return _list(lib().t0b_standard_configs)


def _select(fn, a: int, b: int, c: int) -> GemmConfig:
    out = GemmConfigC()
    if fn(a, b, c, C.byref(out)) != 0:
        raise ValueError(f"auto_select: invalid dimensions ({a}, {b}, {c})")
    return GemmConfig.from_c(out)


def auto_select(m: int, k: int, n: int) -> GemmConfig:
    """(M, K, N) order, like the reference."""
    return _select(lib().t0b_auto_select, m, k, n)


def auto_select_source(m: int, k: int, n: int, trans_a: bool = False, trans_b: bool = True, out_dtype: int = 0):
    """The config a config-less GEMM call of this shape, layout and output type runs, and where it came from:
    "tuned" (measured in this process), "table" (the table shipped with the library) or "model" (the cost model)."""
    c = GemmConfigC()
    src = lib().t0b_auto_select_source(m, k, n, int(trans_a), int(trans_b), out_dtype, C.byref(c))
    if src < 0:
        raise ValueError(f"auto_select_source: invalid shape ({m}, {k}, {n})")
    return GemmConfig.from_c(c), ("model", "table", "tuned")[src]


def auto_select_legacy(m: int, k: int, n: int) -> GemmConfig:
    return _select(lib().t0b_auto_select_legacy, m, k, n)


def auto_select_backward_data(m: int, n_orig: int, k_orig: int) -> GemmConfig:
    return _select(lib().t0b_auto_select_backward_data, m, n_orig, k_orig)


def auto_select_backward_weight(m: int, n_orig: int, k_orig: int) -> GemmConfig:
    return _select(lib().t0b_auto_select_backward_weight, m, n_orig, k_orig)


def _grid(fn, cfg: GemmConfig, *dims) -> tuple:
    gx, gy = C.c_uint32(), C.c_uint32()
    if fn(C.byref(cfg.to_c()), *dims, C.byref(gx), C.byref(gy)) != 0:
        # the reference asserts (panics) on a split_k that is not a power of two
        raise AssertionError(f"compute_grid: invalid arguments {dims} for {cfg.name()}")
    return gx.value, gy.value


def compute_grid(cfg: GemmConfig, m: int, n: int) -> tuple:
    return _grid(lib().t0b_compute_grid, cfg, m, n)


def compute_grid_split_k(cfg: GemmConfig, m: int, n: int, split_k: int) -> tuple:
    return _grid(lib().t0b_compute_grid_split_k, cfg, m, n, split_k)


def compute_grid_auto(cfg: GemmConfig, m: int, n: int) -> tuple:
    return _grid(lib().t0b_compute_grid_auto, cfg, m, n)


def compute_grid_backward_data(cfg: GemmConfig, m: int, k_orig: int) -> tuple:
    return _grid(lib().t0b_compute_grid_backward_data, cfg, m, k_orig)


def compute_grid_backward_weight(cfg: GemmConfig, n_orig: int, k_orig: int) -> tuple:
    return _grid(lib().t0b_compute_grid_backward_weight, cfg, n_orig, k_orig)


def _blob(n: int):
    return (C.c_uint8 * n)()


def build_kernargs(x_addr: int, wt_addr: int, y_addr: int, k: int, n: int, m: int, cfg: GemmConfig) -> bytes:
    out = _blob(40)
    lib().t0b_build_kernargs(x_addr, wt_addr, y_addr, k, n, m, C.byref(cfg.to_c()), out)
    return bytes(out)


def build_kernargs_with_bias(x_addr: int, wt_addr: int, y_addr: int, k: int, n: int, m: int, cfg: GemmConfig,
                             bias_addr: int) -> bytes:
    out = _blob(48)
    lib().t0b_build_kernargs_with_bias(x_addr, wt_addr, y_addr, k, n, m, C.byref(cfg.to_c()), bias_addr, out)
    return bytes(out)


def build_kernargs_m(x_addr: int, wt_addr: int, y_addr: int, k: int, n: int, m: int) -> bytes:
    """tile_ir::build_kernargs_m (src/t0/tile_ir.rs:3173-3190): 44 bytes, M at 40..44."""
    out = _blob(44)
    lib().t0b_build_kernargs_m(x_addr, wt_addr, y_addr, k, n, m, out)
    return bytes(out)


def build_kernargs_backward_data(dy_addr: int, w_addr: int, dx_addr: int, m: int, n_orig: int, k_orig: int,
                                 cfg: GemmConfig) -> bytes:
    out = _blob(40)
    lib().t0b_build_kernargs_backward_data(dy_addr, w_addr, dx_addr, m, n_orig, k_orig, C.byref(cfg.to_c()), out)
    return bytes(out)


def build_kernargs_backward_weight(dy_t_addr: int, x_t_addr: int, dw_addr: int, m: int, n_orig: int, k_orig: int,
                                   cfg: GemmConfig) -> bytes:
    out = _blob(40)
    lib().t0b_build_kernargs_backward_weight(dy_t_addr, x_t_addr, dw_addr, m, n_orig, k_orig, C.byref(cfg.to_c()), out)
    return bytes(out)


@dataclass
class GemmPlan:
    bm: int
    bn: int
    bk: int
    cta_group: int
    m_tiles: int
    n_tiles: int
    stages: int
    split_k: int
    kb_per_split: int
    use_tma: bool
    grid: int
    smem_bytes: int


def resolve_plan(cfg: Optional[GemmConfig], m: int, n: int, k: int, trans_a: bool = False, trans_b: bool = True,
                 lda: Optional[int] = None, ldb: Optional[int] = None, num_sms: int = 148) -> GemmPlan:
    """Which sm_100a kernel variant a GemmConfig runs as for this problem."""
    if lda is None:
        lda = m if trans_a else k
    if ldb is None:
        ldb = k if trans_b else n
    p = GemmPlanC()
    cp = C.byref(cfg.to_c()) if cfg is not None else None
    lib().t0b_resolve_plan(cp, m, n, k, int(trans_a), int(trans_b), lda, ldb, num_sms, C.byref(p))
    return GemmPlan(p.bm, p.bn, p.bk, p.cta_group, p.m_tiles, p.n_tiles, p.stages, p.split_k, p.kb_per_split, bool(p.use_tma), p.grid,
                    p.smem_bytes)
