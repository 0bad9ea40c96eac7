"""Embedding lookup and gradient on the GPU against the CPU oracle (src/t0/embedding_kernels.rs:100-124, GPU test
:186-238; Ignis op src/ignis/ops/embedding.rs:25-178).  Both directions are bit-exact: the forward is a copy, the
backward adds each id's rows in ascending token order like the reference's CPU loop."""
import ctypes as C

import numpy as np
import pytest

import oracle
from t0_gpu_b200._lib import lib

pytestmark = pytest.mark.gpu


def run_fwd(rt, table, ids, dim):
    dt, di = rt.upload_f32(table), rt.upload(np.ascontiguousarray(ids, np.uint32))
    out = rt.alloc(max(len(ids) * dim * 4, 16))
    rt._check(lib().t0b_embedding_fwd(rt.handle, dt.gpu_addr(), di.gpu_addr(), out.gpu_addr(), len(ids), dim, table.shape[0], 0))
    return out.read_as(np.float32, len(ids) * dim).reshape(len(ids), dim)


def run_bwd(rt, grad_table, ids, grad_out, dim, scratch=None):
    dg, di, do = rt.upload_f32(grad_table), rt.upload(np.ascontiguousarray(ids, np.uint32)), rt.upload_f32(grad_out)
    s_addr, s_bytes = (scratch.gpu_addr(), scratch.size()) if scratch is not None else (0, 0)
    rt._check(lib().t0b_embedding_bwd(rt.handle, dg.gpu_addr(), di.gpu_addr(), do.gpu_addr(), len(ids), dim, grad_table.shape[0],
                                      s_addr, s_bytes, 0))
    return dg.read_as(np.float32, grad_table.size).reshape(grad_table.shape)


def test_reference_gpu_case(rt):
    """embedding_kernels.rs:186-238: vocab 16, dim 64, ids [3, 7, 0, 12], table[i] = i * 0.01."""
    vocab, dim = 16, 64
    table = (np.arange(vocab * dim, dtype=np.float32) * np.float32(0.01)).reshape(vocab, dim)
    ids = [3, 7, 0, 12]
    assert np.array_equal(run_fwd(rt, table, ids, dim), oracle.embedding_forward(table, ids, dim))


@pytest.mark.parametrize("vocab,dim,tokens", [(3, 3, 3), (50, 7, 33), (1000, 256, 4096), (32000, 4096, 2048), (257, 1030, 513)])
def test_forward_and_backward_bit_exact(rt, vocab, dim, tokens):
    """Any dim (multiples of 4 take the 128-bit path, others the scalar one); ids drawn so that some rows repeat
    many times and some never appear."""
    rng = np.random.Generator(np.random.Philox(vocab * 7 + dim))
    table = rng.standard_normal((vocab, dim), dtype=np.float32)
    ids = np.minimum(rng.zipf(1.3, tokens) - 1, vocab - 1).astype(np.uint32)      # heavy head, long tail
    assert np.array_equal(run_fwd(rt, table, ids, dim), oracle.embedding_forward(table, ids, dim))
    grad_out = rng.standard_normal((tokens, dim), dtype=np.float32)
    start = rng.standard_normal((vocab, dim), dtype=np.float32)                    # accumulates into what is there
    ref = oracle.embedding_backward(start, ids, grad_out, dim)
    got = run_bwd(rt, start, ids, grad_out, dim)
    assert np.array_equal(got, ref)
    untouched = np.setdiff1d(np.arange(vocab), ids)
    assert np.array_equal(got[untouched], start[untouched])
    for _ in range(3):                                                             # and the same bits on every run
        assert np.array_equal(run_bwd(rt, start, ids, grad_out, dim), got)


def test_backward_with_caller_scratch_and_repeated_single_id(rt):
    vocab, dim, tokens = 8, 128, 1000
    ids = np.full(tokens, 5, np.uint32)                                            # one run of 1000 rows
    grad_out = np.random.Generator(np.random.Philox(3)).standard_normal((tokens, dim), dtype=np.float32)
    need = lib().t0b_embedding_bwd_scratch_bytes(tokens)
    assert need >= 4 * tokens * 4
    scratch = rt.alloc(need)
    zeros = np.zeros((vocab, dim), np.float32)
    got = run_bwd(rt, zeros, ids, grad_out, dim, scratch=scratch)
    assert np.array_equal(got, oracle.embedding_backward(zeros, ids, grad_out, dim))
    small = rt.alloc(256)
    dg = rt.upload_f32(zeros)
    rc = lib().t0b_embedding_bwd(rt.handle, dg.gpu_addr(), dg.gpu_addr(), dg.gpu_addr(), tokens, dim, vocab, small.gpu_addr(), 256, 0)
    assert rc == -1 and b"scratch" in lib().t0b_last_error(rt.handle)


def test_out_of_range_id_is_reported_not_dereferenced(rt):
    """The reference does not check ids; here an id >= vocab reads and writes nothing, the output row is zeros and the
    call reports device status 110.  The context stays usable."""
    vocab, dim = 4, 8
    table = np.arange(vocab * dim, dtype=np.float32).reshape(vocab, dim)
    ids = np.array([1, 9, 2], np.uint32)
    dt, di = rt.upload_f32(table), rt.upload(ids)
    out = rt.alloc(3 * dim * 4)
    rc = lib().t0b_embedding_fwd(rt.handle, dt.gpu_addr(), di.gpu_addr(), out.gpu_addr(), 3, dim, vocab, 0)
    assert rc == -4 and rt.device_status(clear=True) == 110 and not rt.is_poisoned()
    got = out.read_as(np.float32, 3 * dim).reshape(3, dim)
    assert np.array_equal(got[0], table[1]) and np.all(got[1] == 0) and np.array_equal(got[2], table[2])
    dg, do = rt.upload_f32(np.zeros((vocab, dim), np.float32)), rt.upload_f32(np.ones((3, dim), np.float32))
    rc = lib().t0b_embedding_bwd(rt.handle, dg.gpu_addr(), di.gpu_addr(), do.gpu_addr(), 3, dim, vocab, 0, 0, 0)
    assert rc == -4 and rt.device_status(clear=True) == 110
    g = dg.read_as(np.float32, vocab * dim).reshape(vocab, dim)
    assert np.all(g[1] == 1) and np.all(g[2] == 1) and np.all(g[0] == 0) and np.all(g[3] == 0)
    assert np.array_equal(run_fwd(rt, table, [0, 3], dim), table[[0, 3]])          # next call is fine
