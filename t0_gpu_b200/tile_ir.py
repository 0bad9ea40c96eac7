"""Host-side mirror of the reference's tile_ir front end (src/t0/tile_ir.rs): `TileGemm` specs with an epilogue
chain, `tile_auto_select`, `compute_grid`, `build_kernargs_m`, `lower_gemm`.  Every function is a thin call into
the C ABI (t0b_tile_*); kernels are precompiled sm_100a variants, so `lower_gemm` returns a descriptor."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field, replace
from typing import List

from ._lib import TileGemmC, lib


class TileTranspose(enum.IntEnum):
    NT = 0   # Y[M,N] = A[M,K] @ B[N,K]^T  (B row-major with pitch K)
    NN = 1   # Y[M,N] = A[M,K] @ B[K,N]    (B row-major with pitch N)


class EpilogueOp(enum.IntEnum):
    """tile_ir::EpilogueOp (src/t0/tile_ir.rs:41-62); values are the C ABI's T0B_EPI_* codes."""
    BiasAdd = 1
    ReLU = 3
    SiLU = 4
    GELU = 5      # x * sigmoid(1.702 x), the form the reference lowers (src/t0/tile_ir.rs:2254-2282)
    Scale = 6
    Abs = 7
    Neg = 8
    Clamp = 9


@dataclass
class TileGemm:
    """struct TileGemm (src/t0/tile_ir.rs:92-117)."""
    tile_m: int
    tile_n: int
    tile_k: int
    wgp_mode: bool = False
    double_buffer: bool = True
    split_k: int = 1
    swap_grid: bool = True
    transpose: TileTranspose = TileTranspose.NT
    acc_swap: bool = False
    epilogue: List[EpilogueOp] = field(default_factory=list)

    def to_c(self) -> TileGemmC:
        if len(self.epilogue) > 4:
            raise ValueError("TileGemm: at most four epilogue operations")
        c = TileGemmC(self.tile_m, self.tile_n, self.tile_k, int(self.wgp_mode), int(self.double_buffer), self.split_k,
                      int(self.swap_grid), int(self.transpose), int(self.acc_swap), len(self.epilogue))
        for i, op in enumerate(self.epilogue):
            c.epilogue[i] = int(op)
        return c

    @staticmethod
    def from_c(c: TileGemmC) -> "TileGemm":
        return TileGemm(c.tile_m, c.tile_n, c.tile_k, bool(c.wgp_mode), bool(c.double_buffer), c.split_k, bool(c.swap_grid),
                        TileTranspose(c.transpose), bool(c.acc_swap), [EpilogueOp(c.epilogue[i]) for i in range(c.n_epilogue)])

    @staticmethod
    def preset(name: str) -> "TileGemm":
        """TileGemm::tile_<name>() (src/t0/tile_ir.rs:119-316), e.g. preset("128x64_k16")."""
        c = TileGemmC()
        if lib().t0b_tile_preset(name.encode(), C.byref(c)) != 0:
            raise KeyError(f"no TileGemm preset named {name!r}")
        return TileGemm.from_c(c)

    def with_(self, **kw) -> "TileGemm":
        return replace(self, **kw)

    # derived quantities, src/t0/tile_ir.rs:370-404
    def n_waves(self) -> int:
        return self.tile_m // 32

    def wg_size(self) -> int:
        return lib().t0b_tile_wg_size(C.byref(self.to_c()))

    def rows_per_wave(self) -> int:
        return self.tile_m // self.n_waves()

    def n_row_blocks(self) -> int:
        return self.rows_per_wave() // 16

    def n_col_tiles(self) -> int:
        return self.tile_n // 16

    def k_sub_steps(self) -> int:
        return self.tile_k // 16

    def lds_total(self) -> int:
        return lib().t0b_tile_lds_total(C.byref(self.to_c()))

    def name(self) -> str:
        buf = C.create_string_buffer(160)
        n = lib().t0b_tile_name(C.byref(self.to_c()), buf, 160)
        if n < 0:
            raise ValueError("TileGemm.name: invalid spec")
        return buf.value.decode()

    # epilogue chain, src/t0/tile_ir.rs:435-458
    def add_epilogue(self, op: EpilogueOp) -> None:
        self.epilogue.append(EpilogueOp(op))

    def with_epilogue(self, ops) -> "TileGemm":
        return replace(self, epilogue=[EpilogueOp(o) for o in ops])

    def has_epilogue_bias(self) -> bool:
        return EpilogueOp.BiasAdd in self.epilogue

    def has_epilogue_scale(self) -> bool:
        return EpilogueOp.Scale in self.epilogue

    def has_epilogue_clamp(self) -> bool:
        return EpilogueOp.Clamp in self.epilogue


def tile_auto_select(m: int, k: int, n: int, transpose: TileTranspose = TileTranspose.NT) -> TileGemm:
    """tile_auto_select(m, k, n, transpose) (src/t0/tile_ir.rs:471-568); argument order (M, K, N)."""
    c = TileGemmC()
    if lib().t0b_tile_auto_select(m, k, n, int(transpose), C.byref(c)) != 0:
        raise ValueError("tile_auto_select: invalid arguments")
    return TileGemm.from_c(c)


def compute_grid(spec: TileGemm, m: int, n: int) -> tuple:
    """tile_ir::compute_grid (src/t0/tile_ir.rs:3193-3202) -> (x threads, y workgroups * split_k, 1)."""
    g = (C.c_uint32 * 3)()
    if lib().t0b_tile_compute_grid(C.byref(spec.to_c()), m, n, g) != 0:
        raise ValueError(f"compute_grid: invalid spec {spec}")
    return (g[0], g[1], g[2])


def build_kernargs_m(x_addr: int, wt_addr: int, y_addr: int, k: int, n: int, m: int, spec: TileGemm, *, bias_addr: int = 0,
                     scale: float = 1.0, clamp_min: float = 0.0, clamp_max: float = 0.0) -> bytes:
    """tile_ir::build_kernargs_m (src/t0/tile_ir.rs:3173-3190): 44 bytes, parameter order (k, n, m); the epilogue
    arguments the lowered kernel declares after M (bias pointer, scale, clamp bounds; :670-682) follow when the
    spec's chain uses them."""
    out = (C.c_uint8 * 80)()
    n_bytes = lib().t0b_tile_build_kernargs(C.byref(spec.to_c()), x_addr, wt_addr, y_addr, k, n, m, bias_addr, scale, clamp_min,
                                            clamp_max, out, 80)
    if n_bytes < 0:
        raise ValueError(f"build_kernargs_m: invalid spec {spec}")
    return bytes(out[:n_bytes])


def build_kernargs(x_addr: int, wt_addr: int, y_addr: int, k: int, n: int, spec: TileGemm) -> bytes:
    """tile_ir::build_kernargs (src/t0/tile_ir.rs:3148-3170): the same blob with M = 0 (a kernel dispatched with it
    masks every row; callers are expected to use build_kernargs_m)."""
    return build_kernargs_m(x_addr, wt_addr, y_addr, k, n, 0, spec)


class TileKernel:
    """What `lower_gemm(&spec)` returns here: a descriptor of the spec; the sm_100a kernels are precompiled."""

    def __init__(self, spec: TileGemm):
        self.spec = spec
        self.name = spec.name()


def lower_gemm(spec: TileGemm) -> TileKernel:
    """tile_ir::lower_gemm (src/t0/tile_ir.rs:585).  Rejects what the reference's lowering asserts on: a tile_k whose
    16-byte chunks per row are not a power of two (:640-655)."""
    chunks = spec.tile_k * 2 // 16
    if chunks == 0 or chunks & (chunks - 1):
        raise ValueError(f"tile_ir: chunks_per_row={chunks} is not a power of 2 for {spec.name()} (tile_k={spec.tile_k})")
    compute_grid(spec, 1, 1)        # validates the spec
    return TileKernel(spec)
