"""tile_ir front end on the host (no GPU): the reference's unit tests for TileGemm (src/t0/tile_ir.rs:2876-2895,
4949-5009), its naming, grid and kernarg layout, and tile_auto_select's branch outcomes worked out by hand from
src/t0/tile_ir.rs:471-568.  (The reference's own test_tile_auto_select, :4385-4407, predates the current table and
no longer agrees with the function; the function is what callers get, so the function is what is pinned here.)"""
import struct

import pytest

from t0_gpu_b200 import tile_ir
from t0_gpu_b200.tile_ir import EpilogueOp, TileGemm, TileTranspose, build_kernargs, build_kernargs_m, compute_grid, lower_gemm, tile_auto_select


def test_tile_gemm_spec_getters():
    s = TileGemm.preset("128x64_k16")                       # tile_ir.rs:2876-2887
    assert (s.n_waves(), s.wg_size(), s.rows_per_wave(), s.n_row_blocks(), s.n_col_tiles(), s.k_sub_steps()) == (4, 128, 32, 2, 4, 1)
    assert s.lds_total() == (128 * 16 * 2 + 64 * 16 * 2) * 2
    s = TileGemm.preset("64x64_k16")                        # :2889-2895
    assert (s.n_waves(), s.n_row_blocks(), s.n_col_tiles()) == (2, 2, 4)
    swap = TileGemm.preset("128x128_k16_swap")
    assert swap.acc_swap and swap.lds_total() == 2 * (128 * 16 * 2) * 2 + 8 * 8 * 32 * 4 * 4


def test_presets_and_names():
    expect = {
        "128x64_k16": "tile_gemm_128x64_k16_db", "64x64_k64": "tile_gemm_64x64_k64_db", "32x64_k16": "tile_gemm_32x64_k16_db",
        "128x128_k32": "tile_gemm_128x128_k32_db_wgp", "128x128_k48": "tile_gemm_128x128_k48_db",
        "128x128_k32_swap": "tile_gemm_128x128_k32_db_swap", "256x64_k32_wgp": "tile_gemm_256x64_k32_db_wgp",
        "256x64_k64_wgp": "tile_gemm_256x64_k64_db_wgp", "128x64_k64": "tile_gemm_128x64_k64_db",
    }
    for preset, name in expect.items():
        assert TileGemm.preset(preset).name() == name
    s = TileGemm.preset("64x64_k16").with_(split_k=4, swap_grid=False, transpose=TileTranspose.NN, double_buffer=False)
    assert s.name() == "tile_gemm_64x64_k16_sk4_mg_nn"
    with pytest.raises(KeyError):
        TileGemm.preset("128x128_k16_wgp")                  # removed in the reference (VGPR budget)


def test_epilogue_chain_names_and_flags():
    s = TileGemm.preset("128x64_k16").with_epilogue([EpilogueOp.BiasAdd, EpilogueOp.ReLU])   # tile_ir.rs:4982-4995
    assert "_bias_relu" in s.name() and s.has_epilogue_bias() and not s.has_epilogue_scale()
    assert TileGemm.preset("64x64_k16").with_epilogue([EpilogueOp.ReLU]).name().endswith("_relu")      # :4949
    assert TileGemm.preset("64x64_k16").with_epilogue([EpilogueOp.SiLU]).name().endswith("_silu")      # :4960
    assert TileGemm.preset("64x64_k16").with_epilogue([EpilogueOp.GELU]).name().endswith("_gelu")      # :4971
    sc = TileGemm.preset("64x64_k16").with_epilogue([EpilogueOp.Scale])                                 # :4998
    assert sc.has_epilogue_scale() and sc.name().endswith("_scale")
    plain = TileGemm.preset("64x64_k16")                                                                # :5011
    assert plain.epilogue == [] and plain.name() == "tile_gemm_64x64_k16_db"
    s2 = TileGemm.preset("64x64_k16")
    s2.add_epilogue(EpilogueOp.Abs); s2.add_epilogue(EpilogueOp.Neg); s2.add_epilogue(EpilogueOp.Clamp)
    assert s2.name() == "tile_gemm_64x64_k16_db_abs_neg_clamp" and s2.has_epilogue_clamp()
    with pytest.raises(ValueError):
        TileGemm.preset("64x64_k16").with_epilogue([EpilogueOp.ReLU] * 5).name()


# (m, k, n) -> (preset, split_k), derived by hand from the function body.
AUTO = [
    ((4096, 4096, 4096), ("128x128_k64", 8)),     # 1024 tiles, 64 K steps -> min(64/8, 8)
    ((1024, 4096, 4096), ("128x128_k64", 8)),
    ((4096, 96, 4096), ("128x128_k32", 1)),       # K % 64 != 0; 3 K steps
    ((4096, 80, 128), ("128x128_k16", 1)),        # 32 tiles -> 4; 80 % 64 and 80 % 32 are non-zero -> no split
    ((2048, 2048, 2048), ("256x64_k32_wgp", 1)),  # WGP with >= 96 tiles never splits
    ((128, 2048, 2048), ("64x64_k32", 8)),        # m < 256; 64 tiles, 64 K steps
    ((2048, 48, 64), ("64x64_k16", 3)),           # K % 32 != 0; 32 tiles -> 4, capped by K/tile_k = 3, and 48 % 48 == 0
    ((512, 512, 512), ("64x64_k64", 1)),          # 64 tiles, 8 K steps
    ((1024, 1024, 1024), ("64x64_k64", 1)),
    ((256, 256, 256), ("64x64_k64", 4)),          # 16 tiles -> 4; 256 % 256 == 0
    ((128, 256, 64), ("64x64_k64", 4)),           # 2 tiles -> 8, capped by K/tile_k = 4
    ((32, 256, 64), ("64x64_k32", 8)),            # min_dim < 64, m >= 32
    ((16, 40, 128), ("32x64_k16", 1)),            # n >= 128, K % 32 != 0; 2 tiles -> 8, cap 2; 40 % 32 != 0 -> no split
    ((16, 256, 64), ("32x64_k16", 8)),            # small everything
]


def _expected_split(preset, m, k, n):
    """The split-K post-pass of tile_auto_select (tile_ir.rs:528-565), restated."""
    s = TileGemm.preset(preset)
    tiles = -(-m // s.tile_m) * -(-n // s.tile_n)
    k_iters = k // s.tile_k
    if s.wgp_mode and tiles >= 96:
        want = 1
    elif tiles < 12:
        want = 8
    elif tiles < 48:
        want = 4
    elif k_iters > 16:
        want = max(1, min(8, k_iters // 8))
    else:
        want = 1
    sk = 1
    if want > 1 and k >= s.tile_k * 2:
        sk = min(want, k // s.tile_k)
        while sk > 1 and k % (s.tile_k * sk) != 0:
            sk //= 2
    return max(sk, 1)


@pytest.mark.parametrize("shape,expect", AUTO)
def test_tile_auto_select_table(shape, expect):
    m, k, n = shape
    preset, split = expect
    got = tile_auto_select(m, k, n)
    want = TileGemm.preset(preset)
    assert (got.tile_m, got.tile_n, got.tile_k, got.wgp_mode) == (want.tile_m, want.tile_n, want.tile_k, want.wgp_mode), got.name()
    assert got.split_k == split == _expected_split(preset, m, k, n), got.name()
    assert k % (got.tile_k * got.split_k) == 0 or got.split_k == 1
    assert tile_auto_select(m, k, n, TileTranspose.NN).transpose == TileTranspose.NN          # tile_ir.rs:4403


def test_tile_auto_select_pinned_splits():
    """A few split_k outcomes written out in full (no helper), including the divisibility back-off."""
    assert tile_auto_select(4096, 4096, 4096).split_k == 8
    assert tile_auto_select(2048, 2048, 2048).split_k == 1
    assert tile_auto_select(256, 256, 256).split_k == 4
    assert tile_auto_select(128, 256, 64).split_k == 4
    assert tile_auto_select(4096, 80, 128).split_k == 1        # want 4; 80 % 64, 80 % 32 both non-zero
    # want 4, capped by K/tile_k = 3, and 48 % (16*3) == 0: the reference returns 3 here, a factor its own lowering
    # then refuses (tile_ir.rs:696 "bad split_k"); the spec is returned as is and refused by compute_grid / dispatch.
    odd = tile_auto_select(2048, 48, 64)
    assert odd.split_k == 3
    with pytest.raises(ValueError):
        compute_grid(odd, 2048, 64)
    assert tile_auto_select(16, 40, 128).split_k == 1          # want 8, cap 2; 40 % 32 != 0


def test_compute_grid():
    s = TileGemm.preset("128x64_k16")
    assert compute_grid(s, 128, 64) == (128, 1, 1)
    assert compute_grid(s, 1000, 768) == (12 * 128, 8, 1)                     # ceil division on both axes
    assert compute_grid(s.with_(swap_grid=False), 1000, 768) == (8 * 128, 12, 1)
    assert compute_grid(s.with_(split_k=4), 256, 256) == (4 * 128, 2 * 4, 1)
    assert compute_grid(tile_auto_select(4096, 4096, 4096), 4096, 4096) == (32 * 128, 32 * 8, 1)
    with pytest.raises(ValueError):
        compute_grid(s.with_(split_k=3), 128, 64)


def test_kernarg_layout():
    s = TileGemm.preset("128x64_k16").with_(split_k=4)
    ka = build_kernargs_m(0x1000, 0x2000, 0x3000, 256, 512, 100, s)
    assert len(ka) == 44
    assert struct.unpack("<QQQIIIII", ka) == (0x1000, 0x2000, 0x3000, 256, 512, 2, 0, 100)   # shift = log2(split_k), stride 0
    assert struct.unpack("<I", build_kernargs(1, 2, 3, 4, 5, s)[40:44]) == (0,)             # tile_ir.rs:3168
    b = build_kernargs_m(1, 2, 3, 4, 5, 6, s.with_epilogue([EpilogueOp.BiasAdd, EpilogueOp.ReLU]), bias_addr=0xABCD0000)
    assert len(b) == 56 and struct.unpack("<Q", b[48:56]) == (0xABCD0000,) and b[44:48] == b"\0\0\0\0"
    c = build_kernargs_m(1, 2, 3, 4, 5, 6, s.with_epilogue([EpilogueOp.Scale, EpilogueOp.Clamp]), scale=0.5, clamp_min=-2.0,
                         clamp_max=3.0)
    assert len(c) == 56 and struct.unpack("<fff", c[44:56]) == (0.5, -2.0, 3.0)
    d = build_kernargs_m(1, 2, 3, 4, 5, 6, s.with_epilogue([EpilogueOp.Clamp, EpilogueOp.BiasAdd, EpilogueOp.Scale]), bias_addr=9,
                         scale=1.5, clamp_min=0.0, clamp_max=6.0)
    # declaration order is fixed (bias, scale, clamp), whatever the order in the chain
    assert len(d) == 68 and struct.unpack("<Q", d[48:56]) == (9,) and struct.unpack("<fff", d[56:68]) == (1.5, 0.0, 6.0)


def test_lower_gemm_rejects_what_the_reference_asserts_on():
    assert lower_gemm(TileGemm.preset("128x128_k32")).name == "tile_gemm_128x128_k32_db_wgp"
    with pytest.raises(ValueError, match="power of 2"):
        lower_gemm(TileGemm.preset("128x128_k48"))           # tile_ir.rs:640-655
    assert tile_ir.TileKernel(TileGemm.preset("64x64_k16")).spec.tile_m == 64
