"""The tile_ir path on the GPU, driven the way the reference's own tests drive it (src/t0/tile_ir.rs:3534-3735,
4249-4380, 5025-5214): spec -> ensure_kernel_t0(name, lower_gemm) -> build_kernargs_m -> compute_grid -> dispatch ->
read_f32, compared with the CPU oracle on the reference's periodic inputs.  The reference's criterion is
|err| <= 0.1 per element; the GEMM tolerances of this repository are applied as well."""
import numpy as np
import pytest

import oracle
from t0_gpu_b200 import T0Error, tile_ir
from t0_gpu_b200.tile_ir import EpilogueOp, TileGemm, TileTranspose, build_kernargs_m, compute_grid, lower_gemm, tile_auto_select

pytestmark = pytest.mark.gpu


def periodic_inputs(m, k, n, scale=1):
    """x[i] = ((i % 17) - 8) * 0.01, wt[i] = ((i % 13) - 6) * 0.01, truncated to bf16 (tile_ir.rs:3542-3543)."""
    x = oracle.periodic_bf16(m * k, 17, 8)
    wt = oracle.periodic_bf16(n * k, 13, 6)
    if scale != 1:       # the epilogue tests use 0.02 (tile_ir.rs:5035-5036): exact doubling in bf16
        x = oracle.f32_to_bf16_trunc(oracle.bf16_to_f32(x) * np.float32(scale))
        wt = oracle.f32_to_bf16_trunc(oracle.bf16_to_f32(wt) * np.float32(scale))
    return x, wt


def run_spec(rt, spec, x, wt, m, k, n, **epi_args):
    xb, wb = rt.upload(x), rt.upload(wt)
    yb = rt.alloc_zero(m * n * 4 * max(1, spec.split_k))         # the reference sizes Y for split_k slabs (tile_ir.rs:3667)
    kernel = rt.ensure_kernel_t0(spec.name(), lambda: lower_gemm(spec), [spec.wg_size(), 1, 1], spec.lds_total())
    ka = build_kernargs_m(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, spec, **epi_args)
    rt.dispatch(kernel, compute_grid(spec, m, n), ka)
    return rt.read_f32(yb, m * n).reshape(m, n)


def check(got, ref, k, x, wt):
    assert np.abs(got - ref).max() <= 0.1                          # the reference's bar
    amax, bmax = np.abs(oracle.bf16_to_f32(x)).max(), np.abs(oracle.bf16_to_f32(wt)).max()
    assert np.abs(got - ref).max() <= 2.0 ** -7 * np.sqrt(k) * amax * bmax
    assert np.linalg.norm(got - ref) <= 5e-3 * np.linalg.norm(ref)


@pytest.mark.parametrize("preset,shape", [("128x64_k16", (128, 64, 64)), ("64x64_k16", (64, 64, 64)),
                                          ("256x64_k32_wgp", (256, 64, 64)), ("256x64_k32_wgp", (512, 256, 256)),
                                          ("128x128_k16_swap", (128, 128, 128))])
def test_single_and_multi_tile_presets(rt, preset, shape):
    """tile_ir.rs:3534-3646 (128x64, 64x64), 4249-4337 (256x64 WGP, one tile and many), 3024-3140 (acc_swap)."""
    m, k, n = shape
    x, wt = periodic_inputs(m, k, n)
    got = run_spec(rt, TileGemm.preset(preset), x, wt, m, k, n)
    check(got, oracle.gemm_bf16(x, wt, m, n, k, threads=8), k, x, wt)


@pytest.mark.parametrize("size", [256, 512, 1024, 2048])
def test_correctness_sweep_with_auto_select(rt, size):
    """tile_ir.rs:3648-3735: square sizes through tile_auto_select, split_k included (256^3 picks split_k = 4)."""
    m = k = n = size
    spec = tile_auto_select(m, k, n, TileTranspose.NT)
    x, wt = periodic_inputs(m, k, n)
    got = run_spec(rt, spec, x, wt, m, k, n)
    rows = np.unique(np.concatenate([np.arange(0, m, max(1, m // 16)), [m - 1]])) if size > 512 else np.arange(m)
    for r in rows:
        ref = oracle.gemm_bf16(x, wt, m, n, k, row_begin=int(r), row_end=int(r) + 1)[r]
        check(got[r], ref, k, x, wt)


@pytest.mark.parametrize("shape", [(33, 100, 50), (129, 65, 17), (100, 300, 200), (1000, 768, 512)])
@pytest.mark.parametrize("transpose", [TileTranspose.NT, TileTranspose.NN])
def test_edges_are_masked_without_padding(rt, shape, transpose):
    """Non-aligned M, N, K (src/t0/test_tile_gemm_suite.rs:190-193) in both layouts; the reference pads its buffers
    for the K tail (:62-99), here the exact-size buffers are enough.  NN reads B[K, N] with pitch N."""
    m, k, n = shape
    x = oracle.rand_bf16(m * k, 7 * m + k)
    wt = oracle.rand_bf16(n * k, 9 * n + k)
    spec = tile_auto_select(m, k, n, transpose).with_(split_k=1)
    b_dev = wt if transpose == TileTranspose.NT else np.ascontiguousarray(wt.reshape(n, k).T).reshape(-1)
    got = run_spec(rt, spec, x, b_dev, m, k, n)
    check(got, oracle.gemm_bf16(x, wt, m, n, k, threads=8), k, x, wt)


def test_multi_dispatch_reuses_the_kernel(rt):
    """tile_ir.rs:4203-4247, 4339-4380: the same kernel dispatched repeatedly gives the same bits."""
    m, k, n = 256, 128, 192
    x, wt = periodic_inputs(m, k, n)
    spec = TileGemm.preset("128x64_k16")
    first = run_spec(rt, spec, x, wt, m, k, n)
    k1 = rt.ensure_kernel_t0(spec.name(), lambda: pytest.fail("the cached kernel must be reused"))
    assert k1.name == spec.name()
    for _ in range(5):
        assert np.array_equal(run_spec(rt, spec, x, wt, m, k, n), first)


def test_epilogues_end_to_end(rt):
    """tile_ir.rs:5025-5214 (ReLU, SiLU, Abs on 64^3 with the 0.02-step inputs) plus the chains that need kernel
    arguments: bias + ReLU, scale, clamp."""
    m = k = n = 64
    x, wt = periodic_inputs(m, k, n, scale=2)
    base = oracle.gemm_bf16(x, wt, m, n, k).astype(np.float64)
    bias = np.linspace(-0.05, 0.05, n).astype(np.float32)
    dbias = rt.upload_f32(bias)
    spec0 = TileGemm.preset("64x64_k16")
    cases = [
        ([EpilogueOp.ReLU], {}, np.maximum(base, 0)),
        ([EpilogueOp.SiLU], {}, base / (1 + np.exp(-base))),
        ([EpilogueOp.Abs], {}, np.abs(base)),
        ([EpilogueOp.GELU], {}, base / (1 + np.exp(-1.702 * base))),
        ([EpilogueOp.Neg], {}, -base),
        ([EpilogueOp.BiasAdd, EpilogueOp.ReLU], {"bias_addr": dbias.gpu_addr()}, np.maximum(base + bias, 0)),
        ([EpilogueOp.Scale], {"scale": -3.0}, base * -3.0),
        ([EpilogueOp.Scale, EpilogueOp.Clamp], {"scale": 10.0, "clamp_min": -0.2, "clamp_max": 0.3}, np.clip(base * 10.0, -0.2, 0.3)),
    ]
    assert (base < 0).sum() > 100 and (base > 0).sum() > 100          # ReLU / Abs have something to do
    for ops, args, ref in cases:
        got = run_spec(rt, spec0.with_epilogue(ops), x, wt, m, k, n, **args)
        assert np.abs(got - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max()), ops
        if ops == [EpilogueOp.Abs]:
            assert (got >= 0).all()
    # fused and separate give the same values (tile_ir.rs:5216-5300 compares the two)
    plain = run_spec(rt, spec0, x, wt, m, k, n)
    fused = run_spec(rt, spec0.with_epilogue([EpilogueOp.ReLU]), x, wt, m, k, n)
    assert np.array_equal(np.maximum(plain, 0), fused)


def test_dispatch_argument_checks(rt):
    m = k = n = 64
    x, wt = periodic_inputs(m, k, n)
    xb, wb, yb = rt.upload(x), rt.upload(wt), rt.alloc(m * n * 4)
    spec = TileGemm.preset("64x64_k16")
    ka = build_kernargs_m(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, spec)
    with pytest.raises(T0Error, match="compute_grid"):
        rt.dispatch(lower_gemm(spec), (128, 1, 1), ka)                      # wrong grid for this M, N
    with pytest.raises(T0Error, match="kernarg blob"):
        rt.dispatch(lower_gemm(spec.with_epilogue([EpilogueOp.Scale])), compute_grid(spec, m, n), ka)   # missing scale
    bias_spec = spec.with_epilogue([EpilogueOp.BiasAdd])
    with pytest.raises(T0Error, match="bias pointer is null"):
        rt.dispatch(lower_gemm(bias_spec), compute_grid(spec, m, n),
                    build_kernargs_m(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, bias_spec))
    with pytest.raises(ValueError):
        lower_gemm(spec.with_(split_k=3))
    assert not rt.is_poisoned()
    rt.dispatch(spec, compute_grid(spec, m, n), ka)                         # a bare TileGemm is accepted too
    assert np.abs(rt.read_f32(yb, m * n).reshape(m, n) - oracle.gemm_bf16(x, wt, m, n, k)).max() <= 0.1
    assert tile_ir.TileKernel(spec).name == "tile_gemm_64x64_k16_db"
