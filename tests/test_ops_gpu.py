"""The Ignis-level ops (matmul forward/backward closures, rmsnorm, cross_entropy) and the low-level
generate -> load -> submit handshake of the reference's examples, against the oracle."""
import numpy as np
import pytest

import oracle
import t0_gpu_b200 as t
from t0_gpu_b200 import ops
from t0_gpu_b200.gpu_context import AqlQueue, DispatchPool, GpuKernel, KernelLoadConfig, KfdDevice, Target, generate

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("m,k,n", [(64, 128, 96), (100, 300, 200), (256, 512, 384)])
def test_matmul_forward_and_backward_closures(rt, m, k, n):
    rng = np.random.default_rng(m + k + n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    xb, wb, dyb = rt.upload_f32(x), rt.upload_f32(w), rt.upload_f32(dy)
    y, backward = ops.matmul(rt, xb, wb, m, k, n)
    x16, w16, dy16 = oracle.f32_to_bf16_rne(x), oracle.f32_to_bf16_rne(w), oracle.f32_to_bf16_rne(dy)
    ref_y = oracle.gemm_bf16(x16, w16, m, n, k, trans_a=False, trans_b=False)
    assert rel_fro(y.read_as(np.float32, m * n).reshape(m, n), ref_y) <= 5e-3
    dx, dw = backward(dyb)
    ref_dx = oracle.gemm_bf16(dy16, w16, m, k, n, trans_a=False, trans_b=True)      # dY * W^T
    ref_dw = oracle.gemm_bf16(x16, dy16, k, n, m, trans_a=True, trans_b=False)      # X^T * dY
    assert rel_fro(dx.read_as(np.float32, m * k).reshape(m, k), ref_dx) <= 5e-3
    assert rel_fro(dw.read_as(np.float32, k * n).reshape(k, n), ref_dw) <= 5e-3


def test_bf16_weight_cache_converts_once_and_a_step_invalidates(rt):
    """GpuRuntime::get_or_create_bf16 / invalidate_bf16 (src/ignis/gpu_context.rs:392-432): two forwards and a backward
    of one Linear convert W once; an optimizer step drops the copy, the next forward converts the new W and matches the
    oracle on the UPDATED weights.  The ops only queue work: nothing is synchronised until a result is read."""
    m, k, n = 64, 256, 128
    rng = np.random.default_rng(11)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    xb, wb, dyb = rt.upload_f32(x), rt.upload_f32(w), rt.upload_f32(dy)
    rt.clear_bf16_cache()
    s0 = rt.bf16_cache_stats()
    l0 = rt.launch_count()
    y1, backward = ops.matmul(rt, xb, wb, m, k, n)
    y2, _ = ops.matmul(rt, xb, wb, m, k, n)
    dx, dw = backward(dyb)
    s1 = rt.bf16_cache_stats()
    assert s1["conversions"] - s0["conversions"] == 1 and s1["hits"] - s0["hits"] == 2 and s1["entries"] == 1
    # launches: 1 weight cast + per op one activation cast (two for dW) and one GEMM = 1 + (1+1) + (1+1) + (1+1) + (2+1)
    assert rt.launch_count() - l0 == 10
    x16, w16, dy16 = oracle.f32_to_bf16_rne(x), oracle.f32_to_bf16_rne(w), oracle.f32_to_bf16_rne(dy)
    ref_y = oracle.gemm_bf16(x16, w16, m, n, k, trans_a=False, trans_b=False)
    got1, got2 = y1.read_as(np.float32, m * n), y2.read_as(np.float32, m * n)
    assert np.array_equal(got1, got2) and rel_fro(got1.reshape(m, n), ref_y) <= 5e-3
    assert rel_fro(dx.read_as(np.float32, m * k).reshape(m, k), oracle.gemm_bf16(dy16, w16, m, k, n, trans_a=False, trans_b=True)) <= 5e-3
    # an optimizer step on W: the cached copy goes, the next forward sees the new weights
    grad = rt.upload_f32(rng.standard_normal((k, n)).astype(np.float32))
    m_s, v_s = rt.alloc_zero(k * n * 4), rt.alloc_zero(k * n * 4)
    ops.adamw_step(rt, wb, grad, m_s, v_s, k * n, 1, lr=0.05)
    assert rt.bf16_cache_stats()["entries"] == 0
    y3, _ = ops.matmul(rt, xb, wb, m, k, n)
    assert rt.bf16_cache_stats()["conversions"] - s1["conversions"] == 1
    w_new = wb.read_as(np.float32, k * n).reshape(k, n)
    assert np.abs(w_new - w).max() > 1e-3
    ref3 = oracle.gemm_bf16(x16, oracle.f32_to_bf16_rne(w_new), m, n, k, trans_a=False, trans_b=False)
    assert rel_fro(y3.read_as(np.float32, m * n).reshape(m, n), ref3) <= 5e-3
    # overwriting the weight buffer from the host also drops its copy
    wb.write(w)
    assert rt.bf16_cache_stats()["entries"] == 0


def test_matmul_with_pretransposed_bf16_weight(rt):
    """bf16_matmul.rs:102-134; shape deliberately not a multiple of any tile (the reference pads, this build masks)."""
    m, k, n = 70, 200, 130
    rng = np.random.default_rng(5)
    x = rng.standard_normal((m, k)).astype(np.float32)
    wt16 = oracle.f32_to_bf16_rne((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
    y = ops.matmul_with_wt_bf16(rt, rt.upload_f32(x), rt.upload(wt16), m, k, n)
    ref = oracle.gemm_bf16(oracle.f32_to_bf16_rne(x), wt16, m, n, k, trans_a=False, trans_b=True)
    assert rel_fro(y.read_as(np.float32, m * n).reshape(m, n), ref) <= 5e-3


def test_embedding_op_closure(rt):
    """`ops::embedding::embedding_forward` + its recorded backward (src/ignis/ops/embedding.rs:25-178)."""
    vocab, dim, seq = 50, 24, 17
    rng = np.random.default_rng(9)
    table = rng.standard_normal((vocab, dim)).astype(np.float32)
    ids = rng.integers(0, vocab, seq).astype(np.uint32)
    out, backward = ops.embedding_forward(rt, rt.upload_f32(table), rt.upload(ids), seq, dim, vocab)
    assert np.array_equal(out.read_as(np.float32, seq * dim).reshape(seq, dim), table[ids])
    go = rng.standard_normal((seq, dim)).astype(np.float32)
    gt = backward(rt.upload_f32(go))
    ref = oracle.embedding_backward(np.zeros((vocab, dim), np.float32), ids, go, dim)
    assert np.array_equal(gt.read_as(np.float32, vocab * dim).reshape(vocab, dim), ref)


def test_rmsnorm_and_cross_entropy_ops(rt):
    rows, dim, V = 6, 2, 11
    x = np.array([[1, 2], [3, 4], [0.5, -1], [2, 2], [-3, 1], [0.1, 0.2]], np.float32)
    g = np.ones(dim, np.float32)
    y, backward = ops.rmsnorm(rt, rt.upload_f32(x), rt.upload_f32(g), rows, dim)
    out = y.read_as(np.float32, rows * dim).reshape(rows, dim)
    assert abs(out[0, 0] - 0.6325) < 1e-3 and abs(out[0, 1] - 1.2649) < 1e-3      # src/ignis/tests.rs:256-267
    ref, _ = oracle.rmsnorm_forward(x, g, ops.RMSNORM_EPS)
    assert np.allclose(out, ref, rtol=1e-4)
    dy = np.random.default_rng(0).standard_normal((rows, dim)).astype(np.float32)
    dx, dg = backward(rt.upload_f32(dy))
    assert np.allclose(dx.read_as(np.float32, rows * dim).reshape(rows, dim), oracle.rmsnorm_backward(dy, x, g, ops.RMSNORM_EPS), rtol=1e-3, atol=1e-5)
    assert np.allclose(dg.read_as(np.float32, dim), oracle.rmsnorm_dgamma(dy, x, ops.RMSNORM_EPS), rtol=1e-3, atol=1e-5)
    logits = np.random.default_rng(1).standard_normal((rows, V)).astype(np.float32)
    targets = np.arange(rows, dtype=np.uint32)
    loss, grad = ops.cross_entropy(rt, rt.upload_f32(logits), rt.upload(targets), rows, V)
    probs = oracle.softmax_forward(logits)
    assert abs(loss - oracle.ce_mean_loss_from_probs(probs, targets)) < 1e-4       # the Ignis loss definition
    assert np.allclose(grad.read_as(np.float32, rows * V).reshape(rows, V), oracle.ce_loss_backward(logits, targets, 1.0 / rows), atol=1e-6)


def test_generate_load_submit_handshake(rt):
    """examples/test_gemm_correctness.rs:93-188 with the runtime objects of this build."""
    cfg = t.GemmConfig.tile_64x64_k16().with_(split_k=4)
    elf = generate(cfg).compile(Target.GFX1100)            # the reference's only target name is accepted
    kernel = GpuKernel.load(rt, elf, KernelLoadConfig(workgroup_size=(cfg.wg_size, 1, 1), lds_size=cfg.lds_total()))
    assert kernel.cfg.name() == cfg.name()
    queue = AqlQueue(rt)
    m, k, n = 128, 1024, 256
    x = oracle.rand_bf16(m * k, m * 1000 + k); wt = oracle.rand_bf16(n * k, n * 2000 + k)
    xb, wb = rt.upload(x), rt.upload(wt)
    yb = rt.alloc_zero(m * n * 4 * 4)
    ka = t.build_kernargs(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, cfg)
    queue.submit(kernel, (*t.compute_grid_split_k(cfg, m, n, 4), 1), ka)
    queue.wait_idle()
    y = oracle.splitk_reduce(yb.read_as(np.float32, m * n * 4), 4).reshape(m, n)
    ref = oracle.gemm_bf16(x, wt, m, n, k)
    assert np.abs(y - ref).max() < 0.01 * k
    with pytest.raises(t.T0Error):
        GpuKernel.load(rt, b"not an elf")


def test_dispatch_bench_times_one_launch(rt):
    """`GpuRuntime::dispatch_bench` (src/ignis/gpu_context.rs:297-307): submit one kernel and wait; here it also returns
    the device time of the launch (CUDA events on the runtime's stream)."""
    cfg = t.GemmConfig.tile_64x64_k16()
    m, k, n = 128, 256, 128
    x = oracle.rand_bf16(m * k, 3); wt = oracle.rand_bf16(n * k, 4)
    xb, wb, yb = rt.upload(x), rt.upload(wt), rt.alloc_zero(m * n * 4)
    ka = t.build_kernargs(xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), k, n, m, cfg)
    ms = rt.dispatch_bench(cfg, t.compute_grid(cfg, m, n), ka)
    assert 0.0 < ms < 50.0
    ref = oracle.gemm_bf16(x, wt, m, n, k)
    assert np.abs(yb.read_as(np.float32, m * n).reshape(m, n) - ref).max() <= 2.0 ** -7 * np.sqrt(k)


def test_example_gemm_correctness_ported_line_for_line(rt):
    """examples/test_gemm_correctness.rs:65-260 with this build's runtime objects standing where the reference's do:
    generate -> compile -> KfdDevice::open -> create_queue -> DispatchPool::new(&device, 32) -> GpuKernel::load ->
    alloc_vram / write -> the 40-byte kernarg blob -> pool.write_kernargs(0, &ka) -> queue.submit -> wait_idle ->
    host-side slab sum in slab order -> max_err < 0.01 * K.  Same configs, sizes, seeds and tolerance."""
    import struct

    G = t.GemmConfig
    configs = [G.tile_64x64_k16(), G.tile_64x64_k32(), G.tile_128x64_k32(), G.tile_128x64_k32().with_(split_k=2),
               G.tile_64x64_k16().with_(split_k=4), G.tile_64x64_k16().with_(split_k=8), G.tile_32x128_k16(),
               G.tile_32x128_k16().with_(split_k=4)]
    sizes = [(64, 64, 64), (128, 128, 128), (256, 256, 256), (64, 256, 64), (128, 1024, 256), (256, 512, 512)]
    compiled = [generate(cfg).compile(Target.GFX1100) for cfg in configs]
    device = KfdDevice.open(rt=rt)
    queue = device.create_queue()
    pool = DispatchPool.new(device, 32)
    assert pool.len() == 32
    gpu_kernels = [GpuKernel.load(device, compiled[ci], KernelLoadConfig(workgroup_size=(cfg.wg_size, 1, 1), lds_size=cfg.lds_total()))
                   for ci, cfg in enumerate(configs)]
    total_tests = total_pass = 0
    for (m, k, n) in sizes:
        x_data = oracle.rand_bf16(m * k, m * 1000 + k)
        wt_data = oracle.rand_bf16(n * k, n * 2000 + k)
        y_ref = oracle.gemm_bf16(x_data, wt_data, m, n, k)
        x_buf, w_buf = device.alloc_vram(m * k * 2), device.alloc_vram(n * k * 2)
        x_buf.write(x_data)
        w_buf.write(wt_data)
        y_bytes = m * n * 4
        for ci, cfg in enumerate(configs):
            sk = cfg.split_k or 1
            effective_n = cfg.tile_n * cfg.n_col_passes
            if m % cfg.tile_m != 0 or n % effective_n != 0 or k % (cfg.tile_k * sk) != 0:
                continue
            total_tests += 1
            grid_x, grid_y = t.compute_grid_split_k(cfg, m, n, sk) if sk > 1 else t.compute_grid(cfg, m, n)
            y_stride = m * n * 4 if sk > 1 else 0
            y_alloc = device.alloc_vram(y_bytes * sk)
            y_alloc.write(np.zeros(y_bytes * sk, np.uint8))
            ka = struct.pack("<QQQIIII", x_buf.gpu_addr(), w_buf.gpu_addr(), y_alloc.gpu_addr(), k, n, 0, y_stride)
            assert ka == t.build_kernargs(x_buf.gpu_addr(), w_buf.gpu_addr(), y_alloc.gpu_addr(), k, n, m, cfg)
            ka_buf = pool.write_kernargs(0, ka)
            queue.submit(gpu_kernels[ci], (grid_x, grid_y, 1), ka_buf)
            queue.wait_idle()
            partials = y_alloc.read_as(np.float32, m * n * sk)
            y_gpu = np.zeros(m * n, np.float32)
            for s in range(sk):                                     # the reference's host-side sum, slab by slab
                y_gpu = y_gpu + partials[s * m * n:(s + 1) * m * n]
            max_err = float(np.abs(y_gpu - y_ref.ravel()).max())
            assert max_err < 0.01 * k, (m, k, n, cfg.name(), max_err)
            # and within this build's own GEMM tolerance
            assert max_err <= 2.0 ** -7 * np.sqrt(k)
            total_pass += 1
            y_alloc.release()
    assert total_tests == total_pass and total_tests >= 30
    # the pool grows on access to any index, like the reference's
    slot = pool.write_kernargs(100, b"\x01" * 40)
    assert pool.len() == 101 and pool.capacity() >= 101 and slot.read() == b"\x01" * 40 and slot.size() == 256
    assert pool.get_kernargs(0).read() == ka_buf.read()
