"""RMSNorm / softmax / cross-entropy / element-wise kernels against the CPU oracle (<= 1e-3 relative), with
the reference's closed-form known answers (src/t0/rmsnorm_kernels.rs:184-208, softmax_kernels.rs:163-183,
ce_loss_kernels.rs:202-215, src/ignis/tests.rs:256-267) and the shapes of the MLP training config
(1024 x 4096 activations, 1024 x 32000 logits)."""
import ctypes as C

import numpy as np
import pytest

import oracle
import t0_gpu_b200 as t
from t0_gpu_b200._lib import lib

pytestmark = pytest.mark.gpu

REL = 1e-3


def rel_err(got, ref):
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def call(rt, fn, *args):
    rt._check(fn(rt.handle, *args))


@pytest.mark.parametrize("rows,cols", [(1, 4), (2, 2), (5, 33), (64, 256), (17, 1000), (128, 4096), (1024, 4096), (3, 8191)])
def test_rmsnorm_forward_backward(rt, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    eps = 1e-6
    xb, wb, dyb = rt.upload_f32(x), rt.upload_f32(w), rt.upload_f32(dy)
    yb, ib, dxb, dgb = rt.alloc(x.nbytes), rt.alloc(rows * 4), rt.alloc(x.nbytes), rt.alloc(cols * 4)
    call(rt, lib().t0b_rmsnorm_fwd, xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), ib.gpu_addr(), rows, cols, eps, 0)
    ref_y, ref_inv = oracle.rmsnorm_forward(x, w, eps)
    assert rel_err(yb.read_as(np.float32, rows * cols).reshape(rows, cols), ref_y) <= REL
    assert rel_err(ib.read_as(np.float32, rows), ref_inv) <= REL
    nbytes = lib().t0b_rmsnorm_bwd_scratch_bytes(rows, cols)
    sb = rt.alloc(nbytes)
    call(rt, lib().t0b_rmsnorm_bwd, dyb.gpu_addr(), xb.gpu_addr(), wb.gpu_addr(), dxb.gpu_addr(), dgb.gpu_addr(),
         sb.gpu_addr(), nbytes, rows, cols, eps, 0)
    assert rel_err(dxb.read_as(np.float32, rows * cols).reshape(rows, cols), oracle.rmsnorm_backward(dy, x, w, eps)) <= REL
    dg = dgb.read_as(np.float32, cols)
    ref_dg = oracle.rmsnorm_dgamma(dy, x, eps)
    assert np.abs(dg - ref_dg).max() <= REL * max(np.abs(ref_dg).max(), 1.0)
    # deterministic: no atomics, so a second run gives the same bits
    call(rt, lib().t0b_rmsnorm_bwd, dyb.gpu_addr(), xb.gpu_addr(), wb.gpu_addr(), dxb.gpu_addr(), dgb.gpu_addr(),
         sb.gpu_addr(), nbytes, rows, cols, eps, 0)
    assert np.array_equal(dg, dgb.read_as(np.float32, cols))
    with pytest.raises(t.T0Error):   # dgamma without enough scratch is rejected
        call(rt, lib().t0b_rmsnorm_bwd, dyb.gpu_addr(), xb.gpu_addr(), wb.gpu_addr(), dxb.gpu_addr(), dgb.gpu_addr(),
             sb.gpu_addr(), 4, rows, cols, eps, 0)


def test_rmsnorm_known_answers(rt):
    x = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    w = np.ones(4, np.float32)
    xb, wb = rt.upload_f32(x), rt.upload_f32(w)
    yb = rt.alloc(64)
    call(rt, lib().t0b_rmsnorm_fwd, xb.gpu_addr(), wb.gpu_addr(), yb.gpu_addr(), 0, 1, 4, 1e-5, 0)
    assert np.allclose(yb.read_as(np.float32, 4), x[0] / np.sqrt(7.5 + 1e-5), atol=1e-5)
    dyb = rt.upload_f32(np.array([1, 0, 0, 0], np.float32))
    dxb = rt.alloc(64)
    call(rt, lib().t0b_rmsnorm_bwd, dyb.gpu_addr(), xb.gpu_addr(), wb.gpu_addr(), dxb.gpu_addr(), 0, 0, 0, 1, 4, 1e-5, 0)
    assert abs(float((dxb.read_as(np.float32, 4) * x[0]).sum())) < 1e-4
    x2 = rt.upload_f32(np.array([[1, 2], [3, 4]], np.float32)); w2 = rt.upload_f32(np.ones(2, np.float32))
    y2 = rt.alloc(64)
    call(rt, lib().t0b_rmsnorm_fwd, x2.gpu_addr(), w2.gpu_addr(), y2.gpu_addr(), 0, 2, 2, 1e-5, 0)
    out = y2.read_as(np.float32, 4)
    assert abs(out[0] - 0.6325) < 1e-3 and abs(out[1] - 1.2649) < 1e-3


@pytest.mark.parametrize("rows,cols", [(2, 4), (4, 32), (7, 257), (64, 256), (9, 5000), (16, 32000), (3, 60001)])
def test_softmax_forward_backward(rt, rows, cols):
    rng = np.random.default_rng(cols)
    x = (4 * rng.standard_normal((rows, cols))).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    xb, dyb = rt.upload_f32(x), rt.upload_f32(dy)
    yb, dxb = rt.alloc(x.nbytes), rt.alloc(x.nbytes)
    call(rt, lib().t0b_softmax_fwd, xb.gpu_addr(), yb.gpu_addr(), rows, cols, 0)
    y = yb.read_as(np.float32, rows * cols).reshape(rows, cols)
    ref = oracle.softmax_forward(x)
    assert rel_err(y, ref) <= REL
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-4)
    call(rt, lib().t0b_softmax_bwd, dyb.gpu_addr(), yb.gpu_addr(), dxb.gpu_addr(), rows, cols, 0)
    dx = dxb.read_as(np.float32, rows * cols).reshape(rows, cols)
    assert rel_err(dx, oracle.softmax_backward(dy, y)) <= REL
    assert np.abs(dx.sum(axis=1)).max() < 1e-4


@pytest.mark.parametrize("rows,cols", [(1, 4), (4, 32), (33, 1000), (8, 4099), (64, 32000), (1024, 32000)])
def test_softmax_cross_entropy(rt, rows, cols):
    rng = np.random.default_rng(rows + cols)
    logits = (3 * rng.standard_normal((rows, cols))).astype(np.float32)
    targets = rng.integers(0, cols, rows).astype(np.uint32)
    scale = 1.0 / rows
    lb, tb = rt.upload_f32(logits), rt.upload(targets)
    lossb, db = rt.alloc(max(rows * 4, 16)), rt.alloc(logits.nbytes)
    call(rt, lib().t0b_softmax_ce, lb.gpu_addr(), tb.gpu_addr(), lossb.gpu_addr(), db.gpu_addr(), rows, cols, cols, scale, 0)
    loss = lossb.read_as(np.float32, rows)
    d = db.read_as(np.float32, rows * cols).reshape(rows, cols)
    ref_loss = oracle.ce_loss_forward(logits, targets)
    ref_d = oracle.ce_loss_backward(logits, targets, scale)
    assert rel_err(loss, ref_loss) <= REL
    assert np.abs(d - ref_d).max() <= REL * np.abs(ref_d).max()
    assert np.abs(d.sum(axis=1)).max() < 1e-5
    # the Ignis form: -mean(ln(max(p[target], 1e-10))) from the probabilities agrees with the mean of the losses
    probs = oracle.softmax_forward(logits)
    assert abs(oracle.ce_mean_loss_from_probs(probs, targets) - float(loss.mean())) <= 1e-3 * max(1.0, abs(float(loss.mean())))
    for b in (lb, tb, lossb, db):
        b.release()


def test_cross_entropy_known_answer(rt):
    lb = rt.upload_f32(np.array([[1.0, 2.0, 3.0, 4.0]], np.float32))
    tb = rt.upload(np.array([2], np.uint32))
    lossb, db = rt.alloc(16), rt.alloc(16)
    call(rt, lib().t0b_softmax_ce, lb.gpu_addr(), tb.gpu_addr(), lossb.gpu_addr(), db.gpu_addr(), 1, 4, 4, 1.0, 0)
    assert abs(lossb.read_as(np.float32, 1)[0] - 1.44019) < 1e-3
    assert abs(db.read_as(np.float32, 4).sum()) < 1e-6


@pytest.mark.parametrize("n", [1, 255, 4096, 1 << 20, (1 << 20) + 3])
def test_elementwise(rt, n):
    rng = np.random.default_rng(n)
    g, u, gr = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    gb, ub, grb = rt.upload_f32(g), rt.upload_f32(u), rt.upload_f32(gr)
    ob, dgb, dub = rt.alloc(max(n * 4, 16)), rt.alloc(max(n * 4, 16)), rt.alloc(max(n * 4, 16))
    call(rt, lib().t0b_silu_gate_fwd, gb.gpu_addr(), ub.gpu_addr(), ob.gpu_addr(), n, 0)
    assert rel_err(ob.read_as(np.float32, n), oracle.silu_gate_forward(g, u)) <= REL
    call(rt, lib().t0b_silu_gate_bwd, grb.gpu_addr(), gb.gpu_addr(), ub.gpu_addr(), dgb.gpu_addr(), dub.gpu_addr(), n, 0)
    rdg, rdu = oracle.silu_gate_backward(gr, g, u)
    assert rel_err(dgb.read_as(np.float32, n), rdg) <= REL and rel_err(dub.read_as(np.float32, n), rdu) <= REL
    call(rt, lib().t0b_residual_add, gb.gpu_addr(), ub.gpu_addr(), n, 0)
    assert np.array_equal(gb.read_as(np.float32, n), oracle.residual_add(g, u))     # one f32 add: exact
    # f32 -> bf16 cast is bit-exact RNE
    cb = rt.alloc(max(n * 2, 16))
    call(rt, lib().t0b_cast_f32_to_bf16, ub.gpu_addr(), cb.gpu_addr(), n, 0)
    assert np.array_equal(cb.read_as(np.uint16, n), oracle.f32_to_bf16_rne(u))
    # AdamW, 3 steps
    p = rng.standard_normal(n).astype(np.float32)
    m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    pb, mb, vb, pbf = rt.upload_f32(p), rt.upload_f32(m), rt.upload_f32(v), rt.alloc(max(n * 2, 16))
    for step in (1, 2, 3):
        call(rt, lib().t0b_adamw_step, pb.gpu_addr(), grb.gpu_addr(), mb.gpu_addr(), vb.gpu_addr(), pbf.gpu_addr(), n,
             1e-3, 0.9, 0.999, 1e-8, 0.01, step, 1.0, 0)
        p, m, v = oracle.adamw_step(p, gr, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, step)
    assert rel_err(pb.read_as(np.float32, n), p) <= REL
    assert np.array_equal(pbf.read_as(np.uint16, n), oracle.f32_to_bf16_rne(pb.read_as(np.float32, n)))


@pytest.mark.parametrize("rows,cols", [(1, 1), (33, 65), (256, 512), (1000, 130)])
def test_cast_transpose(rt, rows, cols):
    x = np.random.default_rng(1).standard_normal((rows, cols)).astype(np.float32)
    xb = rt.upload_f32(x)
    ob = rt.alloc(max(rows * cols * 2, 16))
    call(rt, lib().t0b_cast_f32_to_bf16_transpose, xb.gpu_addr(), ob.gpu_addr(), rows, cols, 0)
    got = ob.read_as(np.uint16, rows * cols).reshape(cols, rows)
    assert np.array_equal(got, oracle.f32_to_bf16_rne(x).T)


@pytest.mark.parametrize("rows,cols", [(1024, 4096), (64, 1024), (37, 2052), (5, 8192), (16, 260), (3, 33), (9, 9000)])
def test_fused_rmsnorm_silu_matches_the_unfused_sequence(rt, rows, cols):
    """t0b_rmsnorm_silu_fwd / _bwd against (a) the sequence of calls they replace -- same bits -- and (b) the oracle
    chain RMSNorm -> SiLU (src/t0/rmsnorm_kernels.rs:140-174, src/ignis/ops/silu.rs:118-130) at the row-kernel
    tolerance.  Shapes cover the register-resident path (cols % 4 == 0, 1024..8192) and the fallback."""
    L = lib()
    rng = np.random.default_rng(rows * 13 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32) * 1.5
    w = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    dh = rng.standard_normal((rows, cols)).astype(np.float32)
    eps = 1e-6
    n = rows * cols
    dx_, dw_, ddh = rt.upload_f32(x), rt.upload_f32(w), rt.upload_f32(dh)
    # unfused forward
    r, a, h16 = rt.alloc(n * 4), rt.alloc(n * 4), rt.alloc(n * 2)
    call(rt, L.t0b_rmsnorm_fwd, dx_.gpu_addr(), dw_.gpu_addr(), r.gpu_addr(), 0, rows, cols, eps, 1)
    call(rt, L.t0b_silu_gate_fwd, r.gpu_addr(), 0, a.gpu_addr(), n, 1)
    call(rt, L.t0b_cast_f32_to_bf16, a.gpu_addr(), h16.gpu_addr(), n, 0)
    want_h = h16.read_as(np.uint16, n)
    # fused forward
    f16, inv = rt.alloc(n * 2), rt.alloc(max(rows * 4, 16))
    call(rt, L.t0b_rmsnorm_silu_fwd, dx_.gpu_addr(), dw_.gpu_addr(), f16.gpu_addr(), inv.gpu_addr(), rows, cols, eps, 0)
    got_h = f16.read_as(np.uint16, n)
    assert np.array_equal(got_h, want_h)
    y_ref, inv_ref = oracle.rmsnorm_forward(x, w, eps)
    silu_ref = oracle.silu_gate_forward(y_ref, np.ones_like(y_ref))
    assert rel_err(oracle.bf16_to_f32(got_h).reshape(rows, cols), silu_ref) <= 2.0 ** -8 + REL      # bf16 rounding of the output
    assert rel_err(inv.read_as(np.float32, rows), np.asarray(inv_ref).reshape(-1)) <= REL
    # unfused backward
    dr, dz, dz16, dg = rt.alloc(n * 4), rt.alloc(n * 4), rt.alloc(n * 2), rt.alloc(max(cols * 4, 16))
    sb = L.t0b_rmsnorm_bwd_scratch_bytes(rows, cols)
    scratch = rt.alloc(sb)
    call(rt, L.t0b_silu_gate_bwd, ddh.gpu_addr(), r.gpu_addr(), 0, dr.gpu_addr(), 0, n, 1)
    call(rt, L.t0b_rmsnorm_bwd, dr.gpu_addr(), dx_.gpu_addr(), dw_.gpu_addr(), dz.gpu_addr(), dg.gpu_addr(), scratch.gpu_addr(), sb,
         rows, cols, eps, 1)
    call(rt, L.t0b_cast_f32_to_bf16, dz.gpu_addr(), dz16.gpu_addr(), n, 0)
    want_dz, want_dg = dz16.read_as(np.uint16, n), dg.read_as(np.float32, cols)
    # fused backward
    fz16, fg = rt.alloc(n * 2), rt.alloc(max(cols * 4, 16))
    call(rt, L.t0b_rmsnorm_silu_bwd, ddh.gpu_addr(), dx_.gpu_addr(), dw_.gpu_addr(), fz16.gpu_addr(), fg.gpu_addr(), scratch.gpu_addr(),
         sb, rows, cols, eps, 0)
    assert np.array_equal(fz16.read_as(np.uint16, n), want_dz)
    assert np.array_equal(fg.read_as(np.float32, cols), want_dg)
    dgate_ref, _ = oracle.silu_gate_backward(dh, y_ref, np.ones_like(y_ref))
    dx_ref = oracle.rmsnorm_backward(dgate_ref, x, w, eps)
    assert rel_err(oracle.bf16_to_f32(fz16.read_as(np.uint16, n)).reshape(rows, cols), dx_ref) <= 2.0 ** -8 + REL
    assert rel_err(fg.read_as(np.float32, cols), oracle.rmsnorm_dgamma(dgate_ref, x, eps)) <= REL
    # dx only (no dgamma, no scratch)
    fz2 = rt.alloc(n * 2)
    call(rt, L.t0b_rmsnorm_silu_bwd, ddh.gpu_addr(), dx_.gpu_addr(), dw_.gpu_addr(), fz2.gpu_addr(), 0, 0, 0, rows, cols, eps, 0)
    assert rel_err(oracle.bf16_to_f32(fz2.read_as(np.uint16, n)).reshape(rows, cols), dx_ref) <= 2.0 ** -8 + REL


@pytest.mark.parametrize("rows,cols", [(4, 32), (33, 1000), (8, 4099), (64, 32000), (1024, 32000)])
def test_softmax_cross_entropy_bf16_gradient(rt, rows, cols):
    """t0b_softmax_ce_bf16 stores the gradient of t0b_softmax_ce rounded to bf16 (RNE): same bits as ce + cast."""
    L = lib()
    rng = np.random.default_rng(cols + rows)
    logits = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    targets = rng.integers(0, cols, rows).astype(np.uint32)
    dl, dt = rt.upload_f32(logits), rt.upload(targets)
    loss1, loss2 = rt.alloc(max(rows * 4, 16)), rt.alloc(max(rows * 4, 16))
    g32, g16a, g16b = rt.alloc(rows * cols * 4), rt.alloc(rows * cols * 2), rt.alloc(rows * cols * 2)
    scale = 1.0 / rows
    call(rt, L.t0b_softmax_ce, dl.gpu_addr(), dt.gpu_addr(), loss1.gpu_addr(), g32.gpu_addr(), rows, cols, cols, scale, 1)
    call(rt, L.t0b_cast_f32_to_bf16, g32.gpu_addr(), g16a.gpu_addr(), rows * cols, 0)
    call(rt, L.t0b_softmax_ce_bf16, dl.gpu_addr(), dt.gpu_addr(), loss2.gpu_addr(), g16b.gpu_addr(), rows, cols, cols, scale, 0)
    assert np.array_equal(g16a.read_as(np.uint16, rows * cols), g16b.read_as(np.uint16, rows * cols))
    assert np.array_equal(loss1.read_as(np.float32, rows), loss2.read_as(np.float32, rows))
    ref = oracle.ce_loss_backward(logits, targets, scale)
    got = oracle.bf16_to_f32(g16b.read_as(np.uint16, rows * cols)).reshape(rows, cols)
    assert np.abs(got - ref).max() <= (2.0 ** -8 + REL) * np.abs(ref).max()
