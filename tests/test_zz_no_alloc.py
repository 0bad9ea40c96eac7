"""The allocation-free RMSNorm backward entry point.

`t0b_rmsnorm_bwd_noalloc` serves callers that cannot obtain device scratch themselves (a runtime whose device
budget was handed out as fixed buffers at start-up; a step loop that must not pay the device-wide
synchronisation of cudaMalloc / cudaFree).  Its scratch is a fixed 2 MiB array inside the library image.  This
test calls it through the C ABI twice in a row -- the second time on a smaller, different problem, so anything
left in the shared array by the first call would show -- and compares dx and dgamma first with the CPU oracle
(the reference's RMSNorm backward formulas) and then with the regular entry point (`t0b_rmsnorm_bwd` with
caller-provided scratch), within the 1e-3 relative tolerance of the row-kernel tests; where both entry points run
the same kernels (fewer than 1024 columns) the two must agree bit for bit.  It also checks that a problem beyond
the built-in scratch is refused with a clear message and that an empty batch gives a zero dgamma.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

import oracle
import t0_gpu_b200 as t
from t0_gpu_b200._lib import lib

pytestmark = pytest.mark.gpu

REL = 1e-3


def _both_ways(rt, rows, cols, seed, same_kernels=False):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    eps = 1e-6
    L = lib()
    xb, wb, dyb = rt.upload_f32(x), rt.upload_f32(w), rt.upload_f32(dy)
    # regular entry point, scratch from the caller
    dx_ref, dg_ref = rt.alloc(x.nbytes), rt.alloc(cols * 4)
    nbytes = L.t0b_rmsnorm_bwd_scratch_bytes(rows, cols)
    sb = rt.alloc(nbytes)
    rt._check(L.t0b_rmsnorm_bwd(rt.handle, dyb.gpu_addr(), xb.gpu_addr(), wb.gpu_addr(), dx_ref.gpu_addr(),
                                dg_ref.gpu_addr(), sb.gpu_addr(), nbytes, rows, cols, eps, 0))
    # allocation-free entry point; outputs pre-filled so a skipped store would show
    dx_new, dg_new = rt.alloc(x.nbytes), rt.alloc(cols * 4)
    dx_new.write(np.full(rows * cols, 123.0, np.float32))
    dg_new.write(np.full(cols, 123.0, np.float32))
    rt._check(L.t0b_rmsnorm_bwd_noalloc(rt.handle, dyb.gpu_addr(), xb.gpu_addr(), wb.gpu_addr(), dx_new.gpu_addr(),
                                        dg_new.gpu_addr(), rows, cols, eps, 0))
    a_dx, b_dx = dx_ref.read_as(np.float32, rows * cols), dx_new.read_as(np.float32, rows * cols)
    a_dg, b_dg = dg_ref.read_as(np.float32, cols), dg_new.read_as(np.float32, cols)
    # first against the oracle ...
    o_dx = oracle.rmsnorm_backward(dy, x, w, eps).reshape(-1)
    o_dg = oracle.rmsnorm_dgamma(dy, x, eps)
    assert np.abs(b_dx - o_dx).max() <= REL * np.abs(o_dx).max()
    assert np.abs(b_dg - o_dg).max() <= REL * max(np.abs(o_dg).max(), 1.0)
    # ... then against the regular entry point
    assert np.abs(a_dx - b_dx).max() <= REL * np.abs(a_dx).max()
    assert np.abs(a_dg - b_dg).max() <= REL * max(np.abs(a_dg).max(), 1.0)
    if same_kernels:
        assert np.array_equal(a_dx, b_dx) and np.array_equal(a_dg, b_dg)


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice_in_a_row(rt):
    _both_ways(rt, 1024, 4096, seed=1)     # the MLP-step shape; fills most of the shared scratch
    _both_ways(rt, 37, 513, seed=2, same_kernels=True)   # smaller and different: stale scratch contents must not leak in


def test_noalloc_empty_batch_gives_zero_dgamma(rt):
    cols = 256
    buf = rt.alloc(4096)
    dg = rt.alloc(cols * 4)
    dg.write(np.full(cols, 5.0, np.float32))
    rt._check(lib().t0b_rmsnorm_bwd_noalloc(rt.handle, buf.gpu_addr(), buf.gpu_addr(), buf.gpu_addr(), buf.gpu_addr(),
                                            dg.gpu_addr(), 0, cols, 1e-6, 0))      # synchronous: the result is ready on return
    assert not dg.read_as(np.float32, cols).any()


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch(rt):
    buf = rt.alloc(4096)
    rc = lib().t0b_rmsnorm_bwd_noalloc(rt.handle, buf.gpu_addr(), buf.gpu_addr(), buf.gpu_addr(), buf.gpu_addr(),
                                       buf.gpu_addr(), 1024, 8192, 1e-6, 0)     # 1024 + 64*8192 > 524288 floats
    assert rc == -1
    msg = lib().t0b_last_error(rt.handle).decode()
    assert "exceeds the built-in scratch" in msg and "t0b_rmsnorm_bwd" in msg
    assert not rt.is_poisoned()
