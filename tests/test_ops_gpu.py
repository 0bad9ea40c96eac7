"""The Ignis-level ops (matmul forward/backward closures, rmsnorm, cross_entropy) and the low-level
generate -> load -> submit handshake of the reference's examples, against the oracle."""
import numpy as np
import pytest

import oracle
import t0_gpu_b200 as t
from t0_gpu_b200 import ops
from t0_gpu_b200.gpu_context import AqlQueue, GpuKernel, KernelLoadConfig, Target, generate

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
