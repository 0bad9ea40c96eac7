"""Runtime behaviour on the GPU: buffer pool, explicit copies, bounded in-kernel waits (failure detection
without faulting the device), CUDA-graph replay of a launch-bound GEMM, on-device tuning."""
import ctypes as C

import numpy as np
import pytest

import oracle
import t0_gpu_b200 as t
from t0_gpu_b200._lib import lib

pytestmark = pytest.mark.gpu


def test_pool_recycles_by_rounded_size(rt):
    before = rt.pool_stats()
    a = rt.alloc(5000)          # rounds to 8192
    addr = a.gpu_addr()
    rt.recycle(a)
    assert rt.pool_stats()["cached_bytes"] == before["cached_bytes"] + 8192
    b = rt.alloc(8000)          # same 4 KiB class: comes back from the pool
    assert b.gpu_addr() == addr
    assert rt.pool_stats()["hits"] == before["hits"] + 1
    data = np.arange(2000, dtype=np.float32)
    b.write(data)
    assert np.array_equal(b.read_as(np.float32, 2000), data)
    with pytest.raises(AssertionError):
        b.write(np.zeros(4000, np.float32))        # larger than the buffer (bounds assert, kfd/mod.rs:962)
    z = rt.alloc_f32(10)
    assert z.size() >= 512 and np.all(z.read_as(np.float32, 10) == 0.0)


def test_bounded_wait_times_out_and_context_survives(rt):
    """A wait on a barrier nothing signals runs out after its limit, the kernel records a status code and
    returns; the context is not poisoned and the next GEMM works."""
    rc = rt.selftest_bounded_wait(20_000_000)       # 20 ms
    assert rc == -4                                  # T0B_ERR_DEVICE
    assert rt.device_status(clear=True) == 105       # DEV_TIMEOUT_SELFTEST
    assert rt.device_status() == 0 and not rt.is_poisoned()
    ones = rt.upload(np.full(64 * 64, 0x3F80, np.uint16))
    c = rt.alloc(64 * 64 * 4)
    rt.gemm(ones, ones, c, 64, 64, 64)
    assert np.all(c.read_as(np.float32, 64 * 64) == 64.0)


def test_graph_replay_of_small_gemm(rt):
    """256^3 is launch-bound; a captured graph of 8 GEMMs replays with one submission."""
    m = n = k = 256
    A = oracle.rand_bf16(m * k, 256 * 1000 + 256)
    B = oracle.rand_bf16(n * k, 256 * 2000 + 256)
    da, db = rt.upload(A), rt.upload(B)
    outs = [rt.alloc(m * n * 4) for _ in range(8)]
    rt.gemm(da, db, outs[0], m, n, k)                 # warm (function attributes, tensor maps) outside capture
    ref = outs[0].read_as(np.float32, m * n)
    rt._check(lib().t0b_graph_begin(rt.handle))
    for o in outs:
        rt.gemm(da, db, o, m, n, k, async_=True)
    h = C.c_uint64()
    rt._check(lib().t0b_graph_end(rt.handle, C.byref(h)))
    for o in outs:
        o.zero()
    rt._check(lib().t0b_graph_launch(rt.handle, h.value, 0))
    for o in outs:
        assert np.array_equal(o.read_as(np.float32, m * n), ref)
    rt._check(lib().t0b_graph_destroy(rt.handle, h.value))


def test_tuner_returns_a_valid_config(rt):
    cfg, tflops = rt.tune(1024, 1024, 1024)
    assert cfg.tile_m in (128, 256) and cfg.tile_n in (64, 128, 256) and tflops > 1.0
    # the tuned choice is what a config-less call now uses, and it is still correct
    A = oracle.rand_bf16(1024 * 1024, 1).reshape(1024, 1024)
    da = rt.upload(A)
    c = rt.alloc(1024 * 1024 * 4)
    rt.gemm(da, da, c, 1024, 1024, 1024)
    ref = oracle.gemm_bf16(A, A, 1024, 1024, 1024, row_begin=5, row_end=6)[5]
    assert np.abs(c.read_as(np.float32, 1024 * 1024).reshape(1024, 1024)[5] - ref).max() < 2 ** -7 * 32


def test_auto_select_prefers_what_this_process_tuned(rt, tmp_path):
    """auto_select's first source is a measurement of this process (GemmTuner's memory cache in the reference,
    src/t0/auto_gemm.rs:91-96); invalidating the shape hands the answer back to the shipped table / cost model."""
    m, n, k = 384, 640, 512            # not a benchmark shape: not in the shipped table
    _, before = t.auto_select_source(m, k, n)
    assert before == "model"
    best, tflops = rt.tune(m, n, k)
    cfg, src = t.auto_select_source(m, k, n)
    assert src == "tuned" and cfg.name() == best.name() and tflops > 0
    assert t.auto_select(m, k, n).name() == best.name()
    lib().t0b_tune_cache_invalidate(str(tmp_path).encode(), m, n, k)
    assert t.auto_select_source(m, k, n)[1] == "model"


def test_launch_counter_counts_kernels(rt):
    a = rt.alloc(64 * 256 * 2); c = rt.alloc(64 * 64 * 4)
    n0 = rt.launch_count()
    rt.gemm(a, a, c, 64, 64, 64, cfg=t.GemmConfig.preset("b200_128x64"))
    assert rt.launch_count() == n0 + 1
    rt.gemm(a, a, c, 64, 64, 256, cfg=t.GemmConfig.preset("b200_128x64").with_(split_k=2))
    assert rt.launch_count() == n0 + 2      # split-K on a single-CTA tile: ONE launch (the cluster sums the partials)
    b = rt.alloc(512 * 256 * 2); c2 = rt.alloc(512 * 512 * 4)
    rt.gemm(b, b, c2, 512, 512, 256, cfg=t.GemmConfig.preset("b200_256x256").with_(split_k=2))
    assert rt.launch_count() == n0 + 4      # split-K on a CTA-pair tile: GEMM into slabs + reduce kernel


def test_gemm_rejects_operands_larger_than_their_buffers(rt):
    """An operand that starts one of the runtime's own allocations must fit in it; the call is refused on the host
    and nothing is launched (the reference asserts the same way on GpuBuffer::write, src/kfd/mod.rs:962-975)."""
    small = rt.alloc(1 << 20); big, big2, big3 = rt.alloc(4 << 20), rt.alloc(4 << 20), rt.alloc(4 << 20)
    n0 = rt.launch_count()
    for args in ((small, big2, big3), (big, small, big3), (big, big2, small)):
        with pytest.raises(t.T0Error, match="does not fit"):
            rt.gemm(args[0], args[1], args[2], 1024, 1024, 1024)
    assert rt.launch_count() == n0 and not rt.is_poisoned()
    rt.gemm(big, big2, big3, 1024, 1024, 1024)               # fitting operands pass


def test_cuda_error_poisons_the_context_and_a_new_one_works():
    """After a CUDA error the runtime refuses further work, like the reference's poisoned queue
    (src/ignis/gpu_context.rs:149-157, 270-287).  The error is produced on the host side: a copy from an address
    the driver knows is not device memory is rejected by the runtime before anything reaches the GPU."""
    r = t.GpuRuntime()
    host = np.zeros(16, np.uint8)
    rc = lib().t0b_memcpy_d2h(r.handle, host.ctypes.data, 0x10, 16)
    assert rc == -2 and r.is_poisoned()                       # T0B_ERR_CUDA
    msg = lib().t0b_last_error(r.handle).decode()
    assert "cudaMemcpyAsync" in msg
    p = C.c_uint64()
    assert lib().t0b_alloc(r.handle, 64, C.byref(p)) == -3    # T0B_ERR_POISONED
    assert lib().t0b_gemm(r.handle, None, 0, 1, 16, 16, 16, 16, 16, 16, 16, 16, 16, 0, 0, 0, 1.0, 0, 0, 0) == -3
    assert lib().t0b_last_error(r.handle).decode() == msg      # the first error's message is kept
    r.close()
    r2 = t.GpuRuntime()                                        # the device itself is fine
    ones = r2.upload(np.full(64 * 64, 0x3F80, np.uint16))
    c = r2.alloc(64 * 64 * 4)
    r2.gemm(ones, ones, c, 64, 64, 64)
    assert np.all(c.read_as(np.float32, 64 * 64) == 64.0)
    r2.close()


def test_gemm_tuner_and_auto_gemm(rt, tmp_path, monkeypatch):
    """GemmTuner::tune + auto_gemm (src/t0/auto_gemm.rs:82-162, 445-480): the first call measures and writes
    <dir>/gemm_MxNxK.json, a fresh tuner on the same directory answers from the file, and auto_gemm runs the
    product with the chosen config."""
    import importlib
    ag = importlib.import_module("t0_gpu_b200.auto_gemm")      # the package also exports the function of that name

    m, n, k = 512, 384, 256
    tuner = ag.GemmTuner.with_cache_dir(str(tmp_path / "at"))
    cfg = tuner.tune(rt, m, n, k)
    res = tuner.cache[(m, n, k)]
    assert not res.from_cache and res.best_tflops > 1.0 and res.all[0][0] == cfg.name()
    assert (tmp_path / "at" / f"gemm_{m}x{n}x{k}.json").exists()
    again = ag.GemmTuner.with_cache_dir(str(tmp_path / "at"))
    cfg2 = again.tune(rt, m, n, k)
    assert again.cache[(m, n, k)].from_cache
    assert (cfg2.tile_m, cfg2.tile_n, cfg2.split_k, cfg2.swap_grid) == (cfg.tile_m, cfg.tile_n, cfg.split_k, cfg.swap_grid)
    monkeypatch.setattr(ag, "_GLOBAL", again)
    A = oracle.rand_bf16(m * k, 31).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 32).reshape(n, k)
    da, db, dc = rt.upload(A), rt.upload(Bt), rt.alloc(m * n * 4)
    tflops = ag.auto_gemm(rt, da, db, dc, m, n, k)
    assert abs(tflops - again.cache[(m, n, k)].best_tflops) < 1e-6
    got = dc.read_as(np.float32, m * n).reshape(m, n)
    ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=8)
    assert np.linalg.norm(got - ref) <= 5e-3 * np.linalg.norm(ref)
    lib().t0b_set_autotune_dir(rt.handle, b"")       # back to the default for the tests that follow


def test_sm_limit_changes_the_grid_not_the_result(rt):
    """t0b_set_sm_limit caps the SMs of the persistent GEMM grids (room for a collective running beside them); the
    tiles are the same, so the product has the same bits."""
    m, n, k = 1024, 1536, 512
    A = oracle.rand_bf16(m * k, 41).reshape(m, k)
    Bt = oracle.rand_bf16(n * k, 42).reshape(n, k)
    da, db, dc = rt.upload(A), rt.upload(Bt), rt.alloc(m * n * 4)
    outs = []
    for limit in (0, 64, 2, 0):
        rt.set_sm_limit(limit)
        for cfg in (None, t.GemmConfig.preset("b200_256x256"), t.GemmConfig.preset("b200_128x128")):
            rt.gemm(da, db, dc, m, n, k, cfg=cfg)
            outs.append(dc.read_as(np.float32, m * n))
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    assert lib().t0b_set_sm_limit(rt.handle, -1) == -1 and lib().t0b_set_sm_limit(rt.handle, 100000) == -1
    rt.set_sm_limit(0)


def test_block_checksums_and_device_copy(rt):
    """t0b_hash_blocks: equal buffers give equal checksums, one changed byte changes exactly its block, swapped words
    change the block too (the words are mixed with their position).  t0b_copy_d2d: dense and pitched copies."""
    n = 3 * 4096 + 512                                  # three full 4 KiB blocks and a short one
    rng = np.random.default_rng(3)
    data = rng.integers(0, 256, n, dtype=np.uint8)
    a, b = rt.upload(data), rt.upload(data)
    nb = 4
    ha, hb = rt.alloc(nb * 16), rt.alloc(nb * 16)
    L = lib()
    rt._check(L.t0b_hash_blocks(rt.handle, a.gpu_addr(), n, 4096, ha.gpu_addr(), 0))
    rt._check(L.t0b_hash_blocks(rt.handle, b.gpu_addr(), n, 4096, hb.gpu_addr(), 0))
    A, B = ha.read_as(np.uint64, 2 * nb), hb.read_as(np.uint64, 2 * nb)
    assert np.array_equal(A, B) and len(set(A.tolist())) == 2 * nb
    changed = data.copy(); changed[4096 + 100] ^= 1
    b.write(changed)
    rt._check(L.t0b_hash_blocks(rt.handle, b.gpu_addr(), n, 4096, hb.gpu_addr(), 0))
    B = hb.read_as(np.uint64, 2 * nb)
    diff = [i for i in range(nb) if not np.array_equal(A[2 * i:2 * i + 2], B[2 * i:2 * i + 2])]
    assert diff == [1]
    swapped = data.copy().view(np.uint64); swapped[[0, 1]] = swapped[[1, 0]]
    b.write(swapped.view(np.uint8))
    rt._check(L.t0b_hash_blocks(rt.handle, b.gpu_addr(), n, 4096, hb.gpu_addr(), 0))
    assert not np.array_equal(A[:2], hb.read_as(np.uint64, 2 * nb)[:2])
    assert L.t0b_hash_blocks(rt.handle, a.gpu_addr(), n + 1, 4096, ha.gpu_addr(), 0) == -1       # sizes in 8-byte units
    # copies: dense, then a 48-byte-wide column block out of rows of 64 bytes into rows of 80 bytes
    src = rng.integers(0, 256, 64 * 32, dtype=np.uint8)
    s_, d_ = rt.upload(src), rt.alloc(64 * 32)
    rt._check(L.t0b_copy_d2d(rt.handle, d_.gpu_addr(), 2048, s_.gpu_addr(), 2048, 2048, 1, 0))
    assert np.array_equal(d_.read_as(np.uint8, 2048), src)
    p_ = rt.alloc(80 * 32); p_.write(np.zeros(80 * 32, np.uint8))
    rt._check(L.t0b_copy_d2d(rt.handle, p_.gpu_addr() + 16, 80, s_.gpu_addr() + 16, 64, 48, 32, 0))
    got = p_.read_as(np.uint8, 80 * 32).reshape(32, 80)
    assert np.array_equal(got[:, 16:64], src.reshape(32, 64)[:, 16:64]) and not got[:, :16].any() and not got[:, 64:].any()
    assert L.t0b_copy_d2d(rt.handle, p_.gpu_addr() + 8, 80, s_.gpu_addr(), 64, 48, 32, 0) == -1  # 16-byte alignment


def test_async_host_copies_are_ordered_with_the_stream(rt):
    """t0b_memcpy_h2d_async / t0b_memcpy2d_d2h_async: the upload is seen by the GEMM queued after it, the read-back sees
    the GEMM queued before it and completes at t0b_sync."""
    import torch

    m = n = k = 256
    A = oracle.rand_bf16(m * k, 1).reshape(m, k); Bt = oracle.rand_bf16(n * k, 2).reshape(n, k)
    a_h = torch.from_numpy(A.view(np.int16).copy()).pin_memory(); b_h = torch.from_numpy(Bt.view(np.int16).copy()).pin_memory()
    c_h = torch.zeros((m, n // 2), dtype=torch.float32).pin_memory()
    a, b, c = rt.alloc(m * k * 2), rt.alloc(n * k * 2), rt.alloc(m * n * 4)
    L = lib()
    rt._check(L.t0b_memcpy_h2d_async(rt.handle, a.gpu_addr(), a_h.data_ptr(), m * k * 2))
    rt._check(L.t0b_memcpy_h2d_async(rt.handle, b.gpu_addr(), b_h.data_ptr(), n * k * 2))
    rt.gemm(a, b, c, m, n, k, async_=True)
    # the right half of C, as a pitched read-back
    rt._check(L.t0b_memcpy2d_d2h_async(rt.handle, c_h.data_ptr(), (n // 2) * 4, c.gpu_addr() + (n // 2) * 4, n * 4, (n // 2) * 4, m))
    rt.synchronize()
    ref = oracle.gemm_bf16(A, Bt, m, n, k, threads=4)
    assert np.abs(c_h.numpy() - ref[:, n // 2:]).max() <= 2.0 ** -7 * np.sqrt(k)
    assert np.array_equal(c_h.numpy(), c.read_as(np.float32, m * n).reshape(m, n)[:, n // 2:])


def test_switching_streams_keeps_pooled_buffers_ordered(rt):
    """A buffer recycled on one stream and handed out again after t0b_ctx_set_stream must not be overwritten while work
    queued on the old stream still reads it: the new stream is ordered behind the old one."""
    import torch

    m = n = k = 1024
    A = oracle.rand_bf16(m * k, 5).reshape(m, k)
    a, c = rt.upload(A), rt.alloc(m * n * 4)
    old = lib().t0b_ctx_stream(rt.handle)
    s2 = torch.cuda.Stream()
    try:
        tmp = rt.alloc(m * k * 2)
        tmp.write(A)
        for _ in range(20):
            rt.gemm(a, tmp, c, m, n, k, async_=True)       # queued on the old stream, reads tmp
        addr = tmp.gpu_addr()
        rt.recycle(tmp)
        rt.set_stream(s2.cuda_stream)
        got = [rt.alloc(m * k * 2) for _ in range(8)]      # the pool hands the same memory out (among others of its size)
        again = [g for g in got if g.gpu_addr() == addr]
        assert again, "the recycled buffer did not come back from the pool"
        rt._check(lib().t0b_memset0(rt.handle, addr, m * k * 2))               # on the NEW stream
        rt.synchronize()
    finally:
        rt.set_stream(old or 0)
    rt.synchronize()
    ref = oracle.gemm_bf16(A, A, m, n, k, row_begin=7, row_end=8)[7]
    assert np.abs(c.read_as(np.float32, m * n).reshape(m, n)[7] - ref).max() <= 2.0 ** -7 * np.sqrt(k)   # not zeros


def test_force_and_dump_config_env():
    """T0_FORCE_CONFIG makes every GEMM without an explicit config run the named preset, T0_DUMP_CONFIG prints one line
    per new shape with the chooser and the kernel variant; the result still matches the oracle."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import numpy as np, oracle, t0_gpu_b200 as t\n"
        "rt = t.GpuRuntime(0)\n"
        "m = n = k = 256\n"
        "A = oracle.rand_bf16(m * k, 11); B = oracle.rand_bf16(n * k, 12)\n"
        "da, db, dc = rt.upload(A), rt.upload(B), rt.alloc(m * n * 4)\n"
        "rt.gemm(da, db, dc, m, n, k)\n"
        "rt.gemm(da, db, dc, m, n, k)\n"
        "ref = oracle.gemm_bf16(A, B, m, n, k, trans_b=True)\n"
        "tol = 2.0 ** -7 * np.sqrt(k) * np.abs(oracle.bf16_to_f32(A)).max() * np.abs(oracle.bf16_to_f32(B)).max()\n"
        "assert np.abs(dc.read_as(np.float32, m * n) - ref.ravel()).max() <= tol   # the GEMM tolerance of the parity suite\n"
        "rt.gemm(da, db, dc, m, n, k, cfg=t.GemmConfig.preset('b200_128x64'))\n"
        "print('ok')\n"
    )
    env = dict(os.environ, T0_FORCE_CONFIG="b200_128x128", T0_DUMP_CONFIG="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]
    lines = [ln for ln in r.stderr.splitlines() if ln.startswith("t0b gemm 256x256x256")]
    assert len(lines) == 2, r.stderr                     # one per (shape, config), not one per call
    assert "(forced) -> tile 128x128" in lines[0]
    assert "(caller) -> tile 128x64" in lines[1]
    # An unknown preset name is an error, not a silent fallback.
    env["T0_FORCE_CONFIG"] = "no_such_tile"
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode != 0 and "T0_FORCE_CONFIG" in (r.stderr + r.stdout)


def test_timeline_build_stamps_in_order():
    """The timeline build of the library (-DT0B_TRACE) stamps the phases of a GEMM launch; the regular build refuses
    t0b_trace_set.  Stamps of one CTA must be ordered: entry <= set-up <= dependency wait <= first issue <= first data <=
    last MMA <= accumulator <= stores <= TMEM freed, and the product is the same as the regular build's."""
    import os

    import torch

    from t0_gpu_b200 import _lib

    rt = t.GpuRuntime(0)
    assert lib().t0b_trace_set(rt.handle, 0, 0) == -6          # T0B_ERR_UNSUPPORTED in the regular build
    if not os.path.exists(_lib.TRACE_LIB_PATH):
        pytest.skip("timeline build not present (python -m t0_gpu_b200.build --trace)")
    L = _lib.load_trace_lib()
    ctx = C.c_void_p()
    assert L.t0b_ctx_create(0, C.byref(ctx)) == 0
    m = n = k = 512
    A = oracle.rand_bf16(m * k, 5)
    B = oracle.rand_bf16(n * k, 6)
    da, db = rt.upload(A), rt.upload(B)
    c_ref, c_tr = rt.alloc(m * n * 4), rt.alloc(m * n * 4)
    rt.gemm(da, db, c_ref, m, n, k)
    trace = torch.zeros(2 * 160 * 16, dtype=torch.int64, device="cuda:0")
    assert L.t0b_trace_set(ctx, trace.data_ptr(), 2) == 0
    for _ in range(2):
        assert L.t0b_gemm(ctx, None, 0, 1, da.gpu_addr(), db.gpu_addr(), c_tr.gpu_addr(), m, n, k, k, k, n, 0, 0, 0, 1.0, 0, 0, 0) == 0
    assert L.t0b_trace_set(ctx, 0, 0) == 0
    tr = trace.cpu().numpy().reshape(2, 160, 16)
    live = tr[1][:, 0] > 0
    assert live.sum() >= 1
    for cta in np.nonzero(live)[0]:
        s = tr[1][cta]
        chain = [s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[8], s[14]]
        assert all(x > 0 for x in chain), (cta, chain)
        assert all(chain[i] <= chain[i + 1] for i in range(len(chain) - 1)), (cta, chain)
        assert s[14] - s[0] < 1_000_000_000           # within a second
    assert np.array_equal(c_tr.read_as(np.float32, m * n), c_ref.read_as(np.float32, m * n))
    L.t0b_ctx_destroy(ctx)
