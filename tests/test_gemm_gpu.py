"""GEMM parity on the GPU, through the C ABI, against the CPU oracle on identical seeded inputs.

Tolerances (bf16 in, f32 accumulate): relative Frobenius error <= 5e-3 and
max |err| <= 2^-7 * sqrt(K) * max|a| * max|b|.  Cases follow the reference's own GPU tests:
examples/test_gemm_correctness.rs (8 configs x 6 shapes, random bf16, split-K slabs summed in order),
examples/test_gemm_backward.rs, src/t0/test_tile_gemm_suite.rs:176-208 (aligned + non-aligned shapes),
src/t0/tile_boundary_tests.rs (sentinels beyond the valid region), examples/hello_gemm_gen.rs (all-ones),
src/t0/precision_vs_torch.rs (torch golden vectors).
"""
import os

import numpy as np
import pytest

import oracle
import t0_gpu_b200 as t
from t0_gpu_b200 import OUT_BF16, OUT_F32, EpilogueOp, GemmConfig

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "torch_ref")


def check(got, ref, k, a_bits, b_bits, extra_abs=0.0):
    amax = float(np.abs(oracle.bf16_to_f32(a_bits)).max())
    bmax = float(np.abs(oracle.bf16_to_f32(b_bits)).max())
    tol_abs = 2.0 ** -7 * np.sqrt(k) * amax * bmax + extra_abs
    err = float(np.abs(got - ref).max())
    rel = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
    assert rel <= 5e-3, f"relative Frobenius error {rel:.3e}"
    assert err <= tol_abs, f"max abs error {err:.3e} > {tol_abs:.3e}"
    return err, rel


def gpu_gemm(rt, A, Bt, *, trans_a=False, trans_b=True, cfg=None, out_dtype=OUT_F32, epilogue=0, bias=None, alpha=1.0):
    """A: logical [M,K] bits, Bt: logical [N,K] bits; stored on the device per trans flags."""
    m, k = A.shape
    n = Bt.shape[0]
    a_dev = np.ascontiguousarray(A.T) if trans_a else A
    b_dev = Bt if trans_b else np.ascontiguousarray(Bt.T)
    da, db = rt.upload(a_dev), rt.upload(b_dev)
    dc = rt.alloc(max(m * n * 4, 16))
    dbias = rt.upload_f32(bias) if bias is not None else None
    rt.gemm(da, db, dc, m, n, k, cfg=cfg, trans_a=trans_a, trans_b=trans_b, out_dtype=out_dtype, epilogue=epilogue,
            bias=dbias, alpha=alpha)
    if out_dtype == OUT_BF16:
        return oracle.bf16_to_f32(dc.read_as(np.uint16, m * n)).reshape(m, n)
    return dc.read_as(np.float32, m * n).reshape(m, n)


# ------------------------------------------------------------------------------------------------ config 1

@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
def test_256_cubed_all_layouts(rt, trans_a, trans_b):
    """M=N=K=256, A and B row-major (NN) plus the A^T / B^T variants, xorshift uniform[-1,1] inputs."""
    m = n = k = 256
    A = oracle.rand_bf16(m * k, m * 1000 + k).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, n * 2000 + k).reshape(n, k)
    ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=8)
    for cfg in (None, GemmConfig.preset("b200_128x128"), GemmConfig.preset("b200_256x128"), GemmConfig.preset("b200_512x256"),
                GemmConfig.preset("b200_256x512")):
        got = gpu_gemm(rt, A, Bt, trans_a=trans_a, trans_b=trans_b, cfg=cfg)
        check(got, ref, k, A, Bt)


# ------------------------------------------------------------------------------------------------ the reference's test matrix

REF_CONFIGS = [
    ("64x64_k16", None), ("64x64_k32", None), ("128x64_k32", None), ("128x64_k32", 2), ("64x64_k16", 4),
    ("64x64_k16", 8), ("32x128_k16", None), ("32x128_k16", 4),
]
REF_SIZES = [(64, 64, 64), (128, 128, 128), (256, 256, 256), (64, 256, 64), (128, 1024, 256), (256, 512, 512)]


def test_reference_correctness_matrix_through_kernarg_dispatch(rt):
    """examples/test_gemm_correctness.rs:61-262 driven the reference's way: compute_grid*, the 40-byte kernarg
    blob, dispatch, then (split-K) the host-side slab sum in slab order."""
    ran = 0
    for (m, k, n) in REF_SIZES:
        x = oracle.rand_bf16(m * k, m * 1000 + k)
        wt = oracle.rand_bf16(n * k, n * 2000 + k)
        ref = oracle.gemm_bf16(x, wt, m, n, k, threads=8)
        xb, wb = rt.upload(x), rt.upload(wt)
        for name, sk in REF_CONFIGS:
            cfg = GemmConfig.preset(name).with_(split_k=sk)
            s = sk or 1
            if m % cfg.tile_m or n % (cfg.tile_n * cfg.n_col_passes) or k % (cfg.tile_k * s):
                continue   # the reference skips shapes its kernels cannot tile
            grid = t.compute_grid_split_k(cfg, m, n, s) if s > 1 else t.compute_grid(cfg, m, n)
            yb = rt.alloc_zero(m * n * 4 * s)
            ka = t.build_kernargs(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, cfg)
            rt.dispatch(cfg, grid, ka)
            if s > 1:
                partials = yb.read_as(np.float32, m * n * s)
                y = np.zeros(m * n, np.float32)
                for i in range(s):
                    y = y + partials[i * m * n:(i + 1) * m * n]
                # identical to the oracle's slab reduce (same order, same f32 adds)
                assert np.array_equal(y, oracle.splitk_reduce(partials, s))
            else:
                y = yb.read_as(np.float32, m * n)
            got = y.reshape(m, n)
            check(got, ref, k, x, wt)
            assert np.abs(got - ref).max() < 0.01 * k      # the reference's own criterion (:240)
            ran += 1
    assert ran >= 30


def test_split_k_slabs_hold_their_k_chunk(rt):
    """Slab s is the partial sum over K chunk s (src/t0/gemm_gen.rs:746-752) when K/sk is a multiple of 64."""
    m, n, k, sk = 128, 192, 1024, 4
    x = oracle.rand_bf16(m * k, 11)
    wt = oracle.rand_bf16(n * k, 12)
    xb, wb = rt.upload(x), rt.upload(wt)
    yb = rt.alloc_zero(m * n * 4 * sk)
    rt.gemm_slabs(xb, wb, yb, m, n, k, sk, cfg=GemmConfig.tile_64x64_k16())
    slabs = yb.read_as(np.float32, m * n * sk).reshape(sk, m, n)
    for s in range(sk):
        ref = oracle.gemm_nt_krange(x, wt, m, n, k, s * k // sk, (s + 1) * k // sk)
        check(slabs[s], ref, k // sk, x, wt)
    # more slabs than 64-wide K blocks: trailing slabs are zero, the sum is still the product
    yb2 = rt.alloc(m * n * 4 * 8)
    yb2.write(np.full(m * n * 8, 7.0, np.float32))
    rt.gemm_slabs(xb, wb, yb2, m, n, 256, 8, cfg=GemmConfig.tile_64x64_k16())
    slabs2 = yb2.read_as(np.float32, m * n * 8).reshape(8, m, n)
    assert np.all(slabs2[4:] == 0.0)


@pytest.mark.parametrize("shape,sk", [((512, 16384, 512), 4), ((512, 16384, 512), 8), ((128, 4096, 4096), None),
                                      ((4096, 4096, 128), None)])
def test_skinny_and_split_k_deterministic(rt, shape, sk):
    """Config 3: skinny shapes and M=N=512, K=16384 with split_k in {4, 8}; the fixed-order reduce makes the
    result bit-identical run to run."""
    m, k, n = shape
    x = oracle.rand_bf16(m * k, m * 1000 + k)
    wt = oracle.rand_bf16(n * k, n * 2000 + k)
    cfg = t.auto_select(m, k, n)
    if sk:
        cfg = cfg.with_(split_k=sk)
    xb, wb = rt.upload(x), rt.upload(wt)
    yb = rt.alloc(m * n * 4)
    rt.gemm(xb, wb, yb, m, n, k, cfg=cfg)
    first = yb.read_as(np.float32, m * n)
    rows = np.unique(np.concatenate([np.arange(0, m, max(1, m // 8)), [m - 1]]))
    for r in rows:   # sampled rows against the oracle (K is large; full check of 512x512x16384 is still cheap per row)
        ref = oracle.gemm_bf16(x, wt, m, n, k, row_begin=int(r), row_end=int(r) + 1)[r]
        check(first.reshape(m, n)[r], ref, k, x, wt)
    for _ in range(9):
        rt.gemm(xb, wb, yb, m, n, k, cfg=cfg)
        assert np.array_equal(first, yb.read_as(np.float32, m * n))
    if sk:
        # the explicit slab path + explicit reduce gives the same bits as the fused call
        slabs = rt.alloc(m * n * 4 * sk)
        rt.gemm_slabs(xb, wb, slabs, m, n, k, sk, cfg=cfg)
        out = rt.alloc(m * n * 4)
        rt.splitk_reduce(slabs, sk, m, n, out)
        assert np.array_equal(first, out.read_as(np.float32, m * n))
        host = oracle.splitk_reduce(slabs.read_as(np.float32, m * n * sk), sk)
        assert np.array_equal(first, host)


# ------------------------------------------------------------------------------------------------ tile_ir behaviour: edges

def make_lcg(n, seed):
    return oracle.lcg_bf16(n, seed)


@pytest.mark.parametrize("m,k,n", [(128, 128, 128), (256, 256, 256), (128, 1024, 512), (256, 512, 128), (512, 512, 512),
                                   (1024, 1024, 1024), (33, 100, 50), (129, 65, 17), (100, 300, 200), (1000, 768, 512)])
def test_tile_suite_shapes_with_padded_k(rt, m, k, n):
    """src/t0/test_tile_gemm_suite.rs:176-208: LCG inputs, K padded to a tile_k multiple with zeros (the row
    pitch), Y padded; dispatched through the 44-byte kernarg blob that carries M."""
    tile_k = 16
    cfg = GemmConfig(tile_m=32 if m % 128 else 128, tile_n=64, tile_k=tile_k, wg_size=32 if m % 128 else 128)
    k_pad = (k + tile_k - 1) // tile_k * tile_k
    x = make_lcg(m * k, 42 + m).reshape(m, k)
    w = make_lcg(n * k, 137 + n).reshape(n, k)
    xp = np.zeros((m, k_pad), np.uint16); xp[:, :k] = x
    m_pad = (m + cfg.tile_m - 1) // cfg.tile_m * cfg.tile_m
    n_pad = (n + cfg.tile_n - 1) // cfg.tile_n * cfg.tile_n
    wp = np.zeros((n_pad, k_pad), np.uint16); wp[:n, :k] = w    # the N kernarg is the padded width
    xb, wb = rt.upload(xp), rt.upload(wp)
    yb = rt.alloc(m_pad * n_pad * 4)
    yb.write(np.full(m_pad * n_pad, -9999.0, np.float32))
    ka = t.build_kernargs_m(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k_pad, n_pad, m)
    rt.dispatch(cfg, t.compute_grid(cfg, m, n), ka)
    y = yb.read_as(np.float32, m_pad * n_pad).reshape(m_pad, n_pad)
    ref = oracle.gemm_bf16(x, w, m, n, k, threads=8)
    check(y[:m, :n], ref, k, x, w)
    # rows beyond M are never stored (tile_boundary_tests.rs:130-146: the sentinel must survive)
    assert np.all(y[m:, :] == -9999.0)


@pytest.mark.parametrize("m,n,k", [(1, 1, 8), (1, 130, 64), (130, 1, 64), (127, 129, 72), (33, 50, 104), (65, 255, 200),
                                   (300, 200, 520), (257, 513, 1032)])
@pytest.mark.parametrize("preset", ["b200_128x64", "b200_128x128", "b200_128x256", "b200_256x128", "b200_256x256",
                                    "b200_512x256", "b200_256x512"])
def test_ragged_edges_without_padding(rt, m, n, k, preset):
    """M, N not multiples of the tile and K not a multiple of 64: TMA zero-fill stands in for the caller's
    padding; nothing outside [M, N] is written (sentinels around the output survive)."""
    A = oracle.rand_bf16(m * k, 5 * m + k).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 7 * n + k).reshape(n, k)
    ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=8)
    ldc = n + 3
    da, db = rt.upload(A), rt.upload(Bt)
    dc = rt.alloc((m + 2) * ldc * 4)
    dc.write(np.full((m + 2) * ldc, -9999.0, np.float32))
    rt.gemm(da, db, dc, m, n, k, cfg=GemmConfig.preset(preset), ldc=ldc)
    full = dc.read_as(np.float32, (m + 2) * ldc).reshape(m + 2, ldc)
    check(full[:m, :n], ref, k, A, Bt)
    assert np.all(full[:m, n:] == -9999.0) and np.all(full[m:] == -9999.0)


def test_unaligned_pitch_uses_cuda_core_kernel(rt):
    """Row pitch not a multiple of 16 bytes (K = 100 unpadded): not TMA-addressable, still correct."""
    for (m, k, n) in [(33, 100, 50), (129, 65, 17), (100, 300, 201)]:
        A = oracle.rand_bf16(m * k, m + k).reshape(m, k)
        Bt = oracle.rand_bf16(n * k, n + k + 1).reshape(n, k)
        assert not t.resolve_plan(None, m, n, k).use_tma or k % 8 == 0
        ref = oracle.gemm_bf16(A, Bt, m, n, k)
        for ta, tb in [(False, True), (False, False), (True, False)]:
            check(gpu_gemm(rt, A, Bt, trans_a=ta, trans_b=tb), ref, k, A, Bt)
        got = gpu_gemm(rt, A, Bt, cfg=GemmConfig.tile_64x64_k16().with_(split_k=2))
        check(got, ref, k, A, Bt)


def test_empty_and_degenerate_shapes(rt):
    a = rt.alloc(1024); b = rt.alloc(1024); c = rt.alloc(1024)
    c.write(np.full(256, 5.0, np.float32))
    rt.gemm(a, b, c, 0, 16, 16)          # M = 0: no-op
    rt.gemm(a, b, c, 16, 0, 16)          # N = 0: no-op
    assert np.all(c.read_as(np.float32, 256) == 5.0)
    rt.gemm(a, b, c, 8, 8, 0)            # K = 0: zeros
    assert np.all(c.read_as(np.float32, 64) == 0.0)
    # K = 0 with a fused store-phase op: the result is epilogue(0), not 0 -- bias, and bias + ReLU (negative entries clamp)
    bias = np.array([1.5, -2.0, 0.25, -0.5, 3.0, 0.0, -1.0, 7.0], np.float32)
    bb = rt.upload_f32(bias)
    rt.gemm(a, b, c, 8, 8, 0, epilogue=int(EpilogueOp.BiasAddStoreF32), bias=bb)
    assert np.array_equal(c.read_as(np.float32, 64).reshape(8, 8), np.tile(bias, (8, 1)))
    rt.gemm(a, b, c, 8, 8, 0, epilogue=int(EpilogueOp.BiasAddReluStoreF32), bias=bb)
    assert np.array_equal(c.read_as(np.float32, 64).reshape(8, 8), np.tile(np.maximum(bias, 0), (8, 1)))
    # K = 0, bf16 output, a row pitch wider than N: only the M x N block is written (one 2-D memset)
    wide = rt.alloc(8 * 16 * 2)
    wide.write(np.full(8 * 16, 0x4000, np.uint16))
    rt.gemm(a, b, wide, 8, 8, 0, ldc=16, out_dtype=OUT_BF16)
    got = wide.read_as(np.uint16, 8 * 16).reshape(8, 16)
    assert np.all(got[:, :8] == 0) and np.all(got[:, 8:] == 0x4000)
    # K = 0 through the unreduced-slab contract: EVERY slab the caller expects is zeroed, not only the first
    slabs = rt.alloc(4 * 8 * 8 * 4)
    slabs.write(np.full(4 * 64, 9.0, np.float32))
    rt.gemm_slabs(a, b, slabs, 8, 8, 0, 4)
    assert np.all(slabs.read_as(np.float32, 4 * 64) == 0.0)


# ------------------------------------------------------------------------------------------------ known answers / goldens

@pytest.mark.parametrize("m,k,n", [(64, 64, 64), (128, 256, 128), (256, 1024, 256), (128, 4096, 512), (512, 512, 512),
                                   (1024, 2048, 1024)])
def test_all_ones_equals_k(rt, m, k, n):
    """examples/hello_gemm_gen.rs:132-135: all-ones bf16 inputs -> every element == K, exactly."""
    ones = np.full(max(m, n) * k, 0x3F80, np.uint16)
    got = gpu_gemm(rt, ones[:m * k].reshape(m, k), ones[:n * k].reshape(n, k), cfg=t.auto_select(m, k, n))
    assert np.all(got == float(k))


def test_torch_golden_vectors(rt):
    """benchmarks/torch_ref: X*W_gate^T, X*W_up^T and swiglu*W_down^T in f32 (precision_vs_torch.rs:302-305
    accepts max_err < 0.05; products of bf16 are exact in f32, so the error here is summation order only)."""
    M, K, N = 64, 256, 512
    ld = lambda name, dt, shape: np.fromfile(os.path.join(GOLD, name), dtype=dt).reshape(shape)
    x = ld("x.bin", np.uint16, (M, K))
    for wn, rn in (("w_gate.bin", "h_gate_f32ref.bin"), ("w_up.bin", "h_up_f32ref.bin")):
        w = ld(wn, np.uint16, (N, K))
        got = gpu_gemm(rt, x, w)
        assert np.abs(got - ld(rn, np.float32, (M, N))).max() < 1e-5
    s = ld("swiglu_bf16_trunc.bin", np.uint16, (M, N))
    wd = ld("w_down.bin", np.uint16, (K, N))
    got = gpu_gemm(rt, s, wd)
    assert np.abs(got - ld("y_bf16_f32acc.bin", np.float32, (M, K))).max() < 1e-5


# ------------------------------------------------------------------------------------------------ epilogues, bf16 output

def test_bias_epilogues_and_kernarg_bias_blob(rt):
    m, k, n = 128, 256, 192
    A = oracle.rand_bf16(m * k, 3).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 4).reshape(n, k)
    bias = np.linspace(-2, 2, n).astype(np.float32)
    base = oracle.gemm_bf16(A, Bt, m, n, k)
    for epi, relu in ((EpilogueOp.BiasAddStoreF32, False), (EpilogueOp.BiasAddReluStoreF32, True)):
        ref = oracle.epilogue_bias(base, bias, relu)
        got = gpu_gemm(rt, A, Bt, epilogue=int(epi), bias=bias)
        assert np.abs(got - ref).max() <= 2.0 ** -7 * np.sqrt(k)
        got_sk = gpu_gemm(rt, A, Bt, epilogue=int(epi), bias=bias, cfg=GemmConfig.tile_64x64_k16().with_(split_k=2))
        assert np.abs(got_sk - ref).max() <= 2.0 ** -7 * np.sqrt(k)
        # the 48-byte blob with a bias pointer (gemm_gen.rs:438-456)
        cfg = GemmConfig.tile_64x64_k16().with_(epilogue=epi)
        xb, wb, bb = rt.upload(A), rt.upload(Bt), rt.upload_f32(bias)
        yb = rt.alloc(m * n * 4)
        ka = t.build_kernargs_with_bias(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, cfg, bb.gpu_addr())
        rt.dispatch(cfg, t.compute_grid_auto(cfg, m, n), ka)
        assert np.abs(yb.read_as(np.float32, m * n).reshape(m, n) - ref).max() <= 2.0 ** -7 * np.sqrt(k)
    with pytest.raises(t.T0Error):
        gpu_gemm(rt, A, Bt, epilogue=int(EpilogueOp.BiasAddStoreF32))   # bias epilogue without a bias


def test_activation_epilogues(rt):
    m, k, n = 128, 128, 128
    A = oracle.rand_bf16(m * k, 8).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 9).reshape(n, k)
    base = oracle.gemm_bf16(A, Bt, m, n, k).astype(np.float64)
    refs = {EpilogueOp.Relu: np.maximum(base, 0), EpilogueOp.SiLU: base / (1 + np.exp(-base)),
            EpilogueOp.GeluSigmoid: base / (1 + np.exp(-1.702 * base)), EpilogueOp.Scale: base * 0.125,
            EpilogueOp.Abs: np.abs(base), EpilogueOp.Neg: -base}
    for epi, ref in refs.items():
        got = gpu_gemm(rt, A, Bt, epilogue=int(epi), alpha=0.125)
        assert np.abs(got - ref).max() <= 1e-3 * max(1.0, np.abs(ref).max()), epi


@pytest.mark.parametrize("preset", ["b200_128x128", "b200_256x256", "b200_512x256", "b200_256x512"])
def test_bf16_output_is_rne_of_f32_result(rt, preset):
    m, k, n = 256, 512, 384
    A = oracle.normal_bf16((m, k), 4321, 1 / np.sqrt(k))
    Bt = oracle.normal_bf16((n, k), 4322, 1 / np.sqrt(k))
    cfg = GemmConfig.preset(preset)
    f32 = gpu_gemm(rt, A, Bt, cfg=cfg, trans_b=False)
    b16 = gpu_gemm(rt, A, Bt, cfg=cfg, trans_b=False, out_dtype=OUT_BF16)
    assert np.array_equal(b16, oracle.bf16_to_f32(oracle.f32_to_bf16_rne(f32)))
    ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=8)
    assert np.linalg.norm(b16 - ref) / np.linalg.norm(ref) <= 5e-3


# ------------------------------------------------------------------------------------------------ backward GEMMs

@pytest.mark.parametrize("m,n,k", [(64, 64, 64), (128, 128, 128), (128, 256, 64), (256, 128, 512), (64, 512, 256),
                                   (256, 256, 256), (128, 64, 1024)])
def test_backward_data_and_weight(rt, m, n, k):
    """examples/test_gemm_backward.rs: forward Y[M,N] = X[M,K] * WT[N,K]^T;
    dX[M,K] = dY[M,N] * WT[N,K] and dW[N,K] = dY^T * X -- without the reference's host transposes: the layout
    flags select how the operands are read."""
    dy = oracle.rand_bf16(m * n, 1 + m).reshape(m, n)
    wt = oracle.rand_bf16(n * k, 2 + n).reshape(n, k)
    x = oracle.rand_bf16(m * k, 3 + k).reshape(m, k)
    # dX: A = dY [M, N_contract], B = WT stored [N_contract, K_out] -> "NN"
    ref_dx = oracle.gemm_bf16(dy, wt, m, k, n, trans_a=False, trans_b=False)
    da, db = rt.upload(dy), rt.upload(wt)
    dc = rt.alloc(m * k * 4)
    rt.gemm(da, db, dc, m, k, n, cfg=t.auto_select_backward_data(m, n, k), trans_a=False, trans_b=False)
    check(dc.read_as(np.float32, m * k).reshape(m, k), ref_dx, n, dy, wt)
    # dW: A = dY stored [M_contract, N] (read transposed), B = X stored [M_contract, K] -> "TN"
    ref_dw = oracle.gemm_bf16(dy, x, n, k, m, trans_a=True, trans_b=False)
    dxb = rt.upload(x)
    dw = rt.alloc(n * k * 4)
    rt.gemm(da, dxb, dw, n, k, m, cfg=t.auto_select_backward_weight(m, n, k), trans_a=True, trans_b=False)
    check(dw.read_as(np.float32, n * k).reshape(n, k), ref_dw, m, dy, x)
    # the reference's route (pre-transposed operands + NT kernel + backward kernargs) gives the same numbers
    cfg = GemmConfig.tile_64x64_k16()
    dyt = rt.upload(oracle.transpose_bf16(dy, m, n)); xt = rt.upload(oracle.transpose_bf16(x, m, k))
    dw2 = rt.alloc(n * k * 4)
    ka = t.build_kernargs_backward_weight(dyt.gpu_addr(), xt.gpu_addr(), dw2.gpu_addr(), m, n, k, cfg)
    rt.dispatch(cfg, t.compute_grid_backward_weight(cfg, n, k), ka)
    check(dw2.read_as(np.float32, n * k).reshape(n, k), ref_dw, m, dy, x)


# ------------------------------------------------------------------------------------------------ config 2 at full size

@pytest.mark.parametrize("n", [2048, 4096, 8192])
def test_square_sweep_full_size_properties(rt, n):
    """M=N=K in {2048, 4096, 8192}, N(0,1)/sqrt(K) inputs, default auto_select.  The oracle checks sampled rows;
    size-independent properties cover the rest: C(A, B1 + B2) = C(A, B1) + C(A, B2) for exactly representable
    B1 + B2 (linearity), and a second run is bit-identical."""
    A = oracle.normal_bf16((n, n), 1234, 1 / np.sqrt(n))
    B = oracle.normal_bf16((n, n), 1235, 1 / np.sqrt(n))       # stored [K, N] (NN)
    da, db = rt.upload(A), rt.upload(B)
    dc = rt.alloc(n * n * 4)
    rt.gemm(da, db, dc, n, n, n, trans_b=False)
    got = dc.read_as(np.float32, n * n).reshape(n, n)
    Bt = np.ascontiguousarray(B.T)
    for r in (0, 1, n // 2 + 3, n - 1):
        ref = oracle.gemm_bf16(A, Bt, n, n, n, row_begin=r, row_end=r + 1, threads=1)[r]
        check(got[r], ref, n, A, B)
    rt.gemm(da, db, dc, n, n, n, trans_b=False)
    assert np.array_equal(got, dc.read_as(np.float32, n * n).reshape(n, n))
    # linearity: B = Bhi + Blo with Bhi keeping the top mantissa bits (both exactly bf16)
    bf = oracle.bf16_to_f32(B)
    hi_bits = (B & np.uint16(0xFFF0)).astype(np.uint16)
    lo = bf - oracle.bf16_to_f32(hi_bits)
    lo_bits = oracle.f32_to_bf16_rne(lo)
    assert np.array_equal(oracle.bf16_to_f32(lo_bits), lo)     # the split is exact
    d1, d2 = rt.upload(hi_bits), rt.upload(lo_bits)
    c1, c2 = rt.alloc(n * n * 4), rt.alloc(n * n * 4)
    rt.gemm(da, d1, c1, n, n, n, trans_b=False)
    rt.gemm(da, d2, c2, n, n, n, trans_b=False)
    s = c1.read_as(np.float32, n * n) + c2.read_as(np.float32, n * n)
    rel = np.linalg.norm(s - got.ravel()) / np.linalg.norm(got)
    assert rel < 1e-5
    for b in (da, db, dc, d1, d2, c1, c2):
        b.release()


# ------------------------------------------------------------------------------------------------ argument validation

def test_bad_arguments_are_rejected_before_launch(rt):
    a = rt.alloc(4096); b = rt.alloc(4096); c = rt.alloc(4096)
    with pytest.raises(t.T0Error):
        rt.gemm(a, b, c, 16, 16, 16, lda=8)                       # pitch shorter than the row
    with pytest.raises(t.T0Error):
        rt.gemm(a, b, c, 16, 16, 16, cfg=GemmConfig.tile_64x64_k16().with_(split_k=3))
    with pytest.raises(t.T0Error):
        rt.gemm(a, b, 0, 16, 16, 16)
    with pytest.raises(t.T0Error):
        rt.gemm(a, b, c, 16, 16, 16, epilogue=99)
    cfg = GemmConfig.tile_64x64_k16()
    with pytest.raises(t.T0Error):
        rt.dispatch(cfg, (64, 1), b"\0" * 41)                      # blob of the wrong size
    with pytest.raises(t.T0Error):
        rt.dispatch(cfg, (65, 1), b"\0" * 40)                      # grid not a multiple of wg_size
    ws = rt.alloc(64)
    with pytest.raises(t.T0Error):
        # undersized workspace (a CTA-pair tile: its split-K goes through slabs; single-CTA tiles need none)
        rt.gemm(a, b, c, 32, 32, 1024, cfg=GemmConfig.preset("b200_256x256").with_(split_k=4), workspace=ws)
    assert not rt.is_poisoned()                                    # validation errors do not poison
    rt.gemm(a, b, c, 16, 16, 16)                                   # and the runtime still works


# ------------------------------------------------------------------------------------------------ config 4 at full size (one GPU)

def test_large_gemm_bf16_output_full_size(rt):
    """M = N = 32768, K = 8192, N(0,1)/sqrt(K) bf16 inputs, bf16 output (2 GiB), on one GPU: sampled rows against the
    oracle, the all-ones known answer on a row block, and bit-identical results for a column block computed alone
    (the property the column-sharded multi-GPU run relies on: no reduction crosses a column block)."""
    import torch
    from t0_gpu_b200._lib import lib

    m = n = 32768
    k = 8192
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev); g.manual_seed(4321)
    a = (torch.randn((m, k), generator=g, device=dev) / k ** 0.5).to(torch.bfloat16)
    g.manual_seed(4322)
    b = (torch.randn((k, n), generator=g, device=dev) / k ** 0.5).to(torch.bfloat16)       # [K, N] row-major
    c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    L = lib()
    rt._check(L.t0b_gemm(rt.handle, None, 0, 0, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, k, n, n, 1, 0, 0, 1.0, 0, 0, 0))
    rows = [0, 777, 16384, m - 1]
    a_np = a[rows].view(torch.uint16).cpu().numpy()
    cols = slice(12288, 12288 + 2048)                                                   # a 2048-column window keeps the oracle cheap
    bt_np = np.ascontiguousarray(b[:, cols].t().contiguous().view(torch.uint16).cpu().numpy())
    ref = oracle.gemm_bf16(a_np, bt_np, len(rows), 2048, k, trans_a=False, trans_b=True, threads=8)
    got = oracle.bf16_to_f32(c[rows][:, cols].contiguous().view(torch.uint16).cpu().numpy())
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 5e-3
    assert np.abs(got - ref).max() <= 2.0 ** -7 * np.sqrt(k) * float(np.abs(oracle.bf16_to_f32(a_np)).max()) * float(np.abs(oracle.bf16_to_f32(bt_np)).max())
    # a column block computed on its own (what one rank of the sharded run does) gives the same bits
    n_local, col0 = 4096, 3 * 4096
    b_blk = b[:, col0:col0 + n_local].contiguous()
    c_blk = torch.zeros((m, n_local), dtype=torch.bfloat16, device=dev)
    rt._check(L.t0b_gemm(rt.handle, None, 0, 0, a.data_ptr(), b_blk.data_ptr(), c_blk.data_ptr(), m, n_local, k, k, n_local, n_local,
                         1, 0, 0, 1.0, 0, 0, 0))
    assert torch.equal(c_blk, c[:, col0:col0 + n_local])
    del a, b, c, b_blk, c_blk
    torch.cuda.empty_cache()


def test_epilogue_chain(rt):
    """tile_ir's epilogue chain (src/t0/tile_ir.rs:41-62, 2213-2339): operations applied in list order."""
    import ctypes as C
    from t0_gpu_b200._lib import lib

    m, k, n = 192, 256, 160
    A = oracle.rand_bf16(m * k, 21).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 22).reshape(n, k)
    bias = np.linspace(-3, 3, n).astype(np.float32)
    base = oracle.gemm_bf16(A, Bt, m, n, k).astype(np.float64)
    da, db, dbias = rt.upload(A), rt.upload(Bt), rt.upload_f32(bias)
    dc = rt.alloc(m * n * 4)
    BIAS, RELU, SILU, GELU, SCALE, ABS, NEG, CLAMP = 1, 3, 4, 5, 6, 7, 8, 9
    cases = [
        ([BIAS, SCALE, RELU], lambda y: np.maximum((y + bias) * 0.5, 0)),
        ([SCALE, BIAS, SILU], lambda y: (y * 0.5 + bias) / (1 + np.exp(-(y * 0.5 + bias)))),
        ([ABS, NEG, CLAMP], lambda y: np.clip(-np.abs(y), -2.0, -0.25)),
        ([BIAS, GELU, SCALE, CLAMP], lambda y: np.clip(((y + bias) / (1 + np.exp(-1.702 * (y + bias)))) * 0.5, -2.0, -0.25)),
        ([], lambda y: y),
    ]
    for ops, fn in cases:
        arr = (C.c_int32 * max(len(ops), 1))(*ops)
        for cfg in (None, GemmConfig.tile_64x64_k16().with_(split_k=2)):      # fused in the GEMM and in the split-K reduce
            cp = C.byref(cfg.to_c()) if cfg is not None else None
            rt._check(lib().t0b_gemm_chain(rt.handle, cp, 0, 1, da.gpu_addr(), db.gpu_addr(), dc.gpu_addr(), m, n, k, k, k, n, 0,
                                           arr, len(ops), dbias.gpu_addr(), 0.5, -2.0, -0.25, 0, 0, 0))
            got = dc.read_as(np.float32, m * n).reshape(m, n)
            ref = fn(base)
            assert np.abs(got - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max()), ops
    too_long = (C.c_int32 * 5)(RELU, ABS, NEG, RELU, ABS)
    assert lib().t0b_gemm_chain(rt.handle, None, 0, 1, da.gpu_addr(), db.gpu_addr(), dc.gpu_addr(), m, n, k, k, k, n, 0, too_long, 5,
                                0, 1.0, 0.0, 0.0, 0, 0, 0) == -1


@pytest.mark.parametrize("m,n,k,ta,tb,chunk", [(1000, 520, 264, False, True, 256), (1000, 520, 264, False, False, 0),
                                               (640, 300, 200, True, False, 128), (2048, 1024, 512, False, False, 512),
                                               (77, 33, 100, False, True, 0), (300, 4100, 136, False, False, 0),
                                               (1100, 2100, 72, True, True, 256), (1536, 1536, 64, False, True, 384)])
def test_host_buffer_gemm_pipeline(rt, m, n, k, ta, tb, chunk):
    """A, B and C in host memory: row blocks of A and column panels of B uploaded alternately, every strip of C
    multiplied and copied back as soon as its operands are resident (more blocks than panels, more panels than
    blocks, one of each)."""
    from t0_gpu_b200._lib import lib

    A = oracle.rand_bf16(m * k, 3 * m + k).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 5 * n + k).reshape(n, k)
    ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=8)
    a_h = np.ascontiguousarray(A.T) if ta else A
    b_h = Bt if tb else np.ascontiguousarray(Bt.T)
    ldc = n + 5
    for out_dtype in (OUT_F32, OUT_BF16):
        c_h = np.full((m, ldc), -9999.0, np.float32) if out_dtype == OUT_F32 else np.full((m, ldc), 0xC61C, np.uint16)
        rt._check(lib().t0b_gemm_host(rt.handle, None, int(ta), int(tb), a_h.ctypes.data, b_h.ctypes.data, c_h.ctypes.data, m, n, k,
                                      a_h.shape[1], b_h.shape[1], ldc, out_dtype, chunk))
        got = c_h[:, :n] if out_dtype == OUT_F32 else oracle.bf16_to_f32(np.ascontiguousarray(c_h[:, :n]))
        if out_dtype == OUT_F32:
            check(got, ref, k, A, Bt)
            assert np.all(c_h[:, n:] == -9999.0)            # the pitch padding of the host C is untouched
            # Another row-block size gives the same bits: the blocking does not change the summation order.
            got = got.copy()
            rt._check(lib().t0b_gemm_host(rt.handle, None, int(ta), int(tb), a_h.ctypes.data, b_h.ctypes.data, c_h.ctypes.data,
                                          m, n, k, a_h.shape[1], b_h.shape[1], ldc, out_dtype, 128 if chunk != 128 else 640))
            assert np.array_equal(c_h[:, :n], got)
        else:
            assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 5e-3
            assert np.all(c_h[:, n:] == 0xC61C)


def test_randomized_shapes_layouts_and_configs(rt):
    """Seeded random draw over what a caller can combine: aligned, 8-aligned and odd shapes (the last take the CUDA-core
    kernel), the four layouts, both output types, no / bias / bias+ReLU epilogue, automatic or explicit tile with
    split-K 2..16 (cluster path, slab path and effective-split clamping all occur) and both raster directions; every
    case against the oracle within the GEMM tolerance."""
    import random

    rnd = random.Random(20240611)
    presets = ["b200_128x64", "b200_128x128", "b200_128x256", "b200_256x128", "b200_256x256", "b200_512x256", "b200_256x512"]
    for case in range(48):
        kind = rnd.random()
        if kind < 0.4:
            m, n, k = rnd.randint(1, 8) * 64, rnd.randint(1, 8) * 64, rnd.randint(1, 10) * 64
        elif kind < 0.8:
            m, n, k = rnd.randint(1, 500), rnd.randint(1, 60) * 8, rnd.randint(1, 80) * 8
        else:
            m, n, k = rnd.randint(1, 300), rnd.randint(1, 300), rnd.randint(1, 300)
        ta, tb = bool(rnd.randint(0, 1)), bool(rnd.randint(0, 1))
        out_dtype = OUT_BF16 if rnd.randint(0, 1) else OUT_F32
        epilogue = rnd.choice([EpilogueOp.StoreF32, EpilogueOp.StoreF32, EpilogueOp.BiasAddStoreF32, EpilogueOp.BiasAddReluStoreF32])
        cfg = None
        if rnd.random() < 0.7:
            cfg = GemmConfig.preset(rnd.choice(presets)).with_(split_k=rnd.choice([None, None, 2, 4, 8, 16]),
                                                              swap_grid=bool(rnd.randint(0, 1)))
        A = oracle.rand_bf16(m * k, 9000 + case).reshape(m, k)
        Bt = oracle.rand_bf16(n * k, 19000 + case).reshape(n, k)
        bias = (np.arange(n, dtype=np.float32) % 7 - 3.0) * 0.25
        ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=8).reshape(m, n)
        if epilogue != EpilogueOp.StoreF32:
            ref = ref + bias[None, :]
        if epilogue == EpilogueOp.BiasAddReluStoreF32:
            ref = np.maximum(ref, 0.0)
        got = gpu_gemm(rt, A, Bt, trans_a=ta, trans_b=tb, cfg=cfg, out_dtype=out_dtype, epilogue=int(epilogue),
                       bias=bias if epilogue != EpilogueOp.StoreF32 else None)
        extra = float(np.abs(ref).max()) * 2.0 ** -8 if out_dtype == OUT_BF16 else 0.0
        try:
            check(got, ref.astype(np.float32), k, A, Bt, extra_abs=extra + 1e-6)
        except AssertionError as e:
            raise AssertionError(f"case {case}: {(m, n, k)} ta={ta} tb={tb} out={out_dtype} epi={epilogue} cfg={cfg and cfg.name()}: {e}")
    assert rt.device_status() == 0
