"""Pin the CPU oracle against the reference's golden vectors and closed-form known answers.

Golden vectors: tests/golden/torch_ref/ (copied from the reference's benchmarks/torch_ref/, the
fixture its src/t0/precision_vs_torch.rs consumes).  Known answers: the reference's CPU unit tests
(ce_loss_kernels.rs:202-215, softmax_kernels.rs:163-183, rmsnorm_kernels.rs:184-208,
ignis/tests.rs:256-267, examples/hello_gemm_gen.rs:132-135).
"""
import hashlib
import json
import os

import numpy as np

import oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "torch_ref")
M, K, N = 64, 256, 512


def _load(name, dtype, shape):
    return np.fromfile(os.path.join(GOLD, name), dtype=dtype).reshape(shape)


def test_fixture_files_unchanged():
    with open(os.path.join(GOLD, "SHA256.json")) as f:
        sums = json.load(f)
    for name, digest in sums.items():
        with open(os.path.join(GOLD, name), "rb") as f:
            assert hashlib.sha256(f.read()).hexdigest() == digest, name


def test_gemm_nt_matches_torch_f32ref():
    """X*W^T on the fixture's bf16 inputs: oracle (sequential f32) vs torch f32 matmul."""
    x = _load("x.bin", np.uint16, (M, K))
    for w_name, ref_name in (("w_gate.bin", "h_gate_f32ref.bin"), ("w_up.bin", "h_up_f32ref.bin")):
        w = _load(w_name, np.uint16, (N, K))
        ref = _load(ref_name, np.float32, (M, N))
        got = oracle.gemm_bf16(x, w, M, N, K, trans_a=False, trans_b=True)
        # Both accumulate exact bf16 products in f32; only the summation order differs.
        assert np.max(np.abs(got - ref)) < 2e-6
        # Exact in float64 to the same bound.
        exact = oracle.bf16_to_f32(x).astype(np.float64) @ oracle.bf16_to_f32(w).astype(np.float64).T
        assert np.max(np.abs(got - exact)) < 2e-6


def test_second_gemm_matches_torch_f32acc():
    s = _load("swiglu_bf16_trunc.bin", np.uint16, (M, N))
    wd = _load("w_down.bin", np.uint16, (K, N))
    ref = _load("y_bf16_f32acc.bin", np.float32, (M, K))
    got = oracle.gemm_bf16(s, wd, M, K, N, trans_a=False, trans_b=True)
    assert np.max(np.abs(got - ref)) < 1e-6


def test_swiglu_trunc_fixture_consistent_with_oracle_casts():
    """swiglu_bf16_trunc is the truncating bf16 cast of silu(h_gate)*h_up (f32 refs)."""
    hg = _load("h_gate_f32ref.bin", np.float32, (M, N))
    hu = _load("h_up_f32ref.bin", np.float32, (M, N))
    s = _load("swiglu_bf16_trunc.bin", np.uint16, (M, N))
    mine = oracle.silu_gate_forward(hg, hu)
    # expf differences may flip the last truncated bit on a few elements; compare as values.
    diff = np.abs(oracle.bf16_to_f32(oracle.f32_to_bf16_trunc(mine)) - oracle.bf16_to_f32(s))
    scale = np.maximum(np.abs(oracle.bf16_to_f32(s)), 1e-3)
    assert np.max(diff / scale) < 2 ** -6


def test_gemm_layout_variants_agree():
    """NN / TN / TT address the same logical matrices -> identical bits."""
    m, n, k = 37, 29, 53
    a = oracle.rand_bf16(m * k, 1).reshape(m, k)
    b = oracle.rand_bf16(n * k, 2).reshape(n, k)  # [N,K]
    nt = oracle.gemm_bf16(a, b, m, n, k, False, True)
    nn = oracle.gemm_bf16(a, np.ascontiguousarray(b.T), m, n, k, False, False)
    tn = oracle.gemm_bf16(np.ascontiguousarray(a.T), np.ascontiguousarray(b.T), m, n, k, True, False)
    tt = oracle.gemm_bf16(np.ascontiguousarray(a.T), b, m, n, k, True, True)
    assert np.array_equal(nt, nn) and np.array_equal(nt, tn) and np.array_equal(nt, tt)
    # threaded == sequential, bit for bit
    assert np.array_equal(nt, oracle.gemm_bf16(a, b, m, n, k, False, True, threads=4))


def test_all_ones_gemm_equals_k():
    for (m, k, n) in [(64, 64, 64), (128, 256, 64), (32, 1024, 128)]:
        ones = np.full(m * k, 0x3F80, dtype=np.uint16)
        w = np.full(n * k, 0x3F80, dtype=np.uint16)
        y = oracle.gemm_bf16(ones, w, m, n, k)
        assert np.all(y == float(k))


def test_splitk_slab_sum_order():
    m, n, k, sk = 16, 24, 256, 4
    x = oracle.rand_bf16(m * k, m * 1000 + k)
    w = oracle.rand_bf16(n * k, n * 2000 + k)
    slabs = np.stack([oracle.gemm_nt_krange(x, w, m, n, k, s * k // sk, (s + 1) * k // sk) for s in range(sk)])
    y = oracle.splitk_reduce(slabs, sk).reshape(m, n)
    acc = np.zeros((m, n), np.float32)
    for s in range(sk):
        acc = acc + slabs[s]
    assert np.array_equal(y, acc)
    full = oracle.gemm_bf16(x, w, m, n, k)
    assert np.max(np.abs(full - y)) < 1e-4


def test_bf16_rounding_modes():
    assert oracle.lib().t0o_f32_to_bf16_rne(1.0) == 0x3F80
    # 1 + 2^-8 is exactly halfway between two bf16 values: ties to even (down)
    assert oracle.f32_to_bf16_rne(np.array([1.00390625], np.float32))[0] == 0x3F80
    # 1 + 3*2^-8 is halfway with odd low bit: rounds up
    assert oracle.f32_to_bf16_rne(np.array([1.01171875], np.float32))[0] == 0x3F82
    assert oracle.f32_to_bf16_trunc(np.array([1.01171875], np.float32))[0] == 0x3F81
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    # RNE cross-check against an independent numpy formulation
    bits = x.view(np.uint32).astype(np.uint64)
    want = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_rne(x), want)


def test_xorshift_generator_against_python_restatement():
    """Independent pure-Python restatement of test_gemm_correctness.rs:45-58."""
    seed = 256 * 1000 + 256
    state = (seed ^ 0xDEADBEEFCAFEBABE) & 0xFFFFFFFFFFFFFFFF
    want = []
    for _ in range(64):
        state ^= (state << 13) & 0xFFFFFFFFFFFFFFFF
        state ^= state >> 7
        state ^= (state << 17) & 0xFFFFFFFFFFFFFFFF
        f = np.float32(np.float32(state >> 32) / np.float32(4294967295)) * np.float32(2.0) - np.float32(1.0)
        want.append(int(oracle.f32_to_bf16_rne(np.array([f], np.float32))[0]))
    got = oracle.rand_bf16(64, seed)
    assert list(got) == want
    vals = oracle.bf16_to_f32(oracle.rand_bf16(10000, 7))
    assert vals.min() >= -1.0 and vals.max() <= 1.0 and abs(vals.mean()) < 0.05


def test_lcg_and_periodic_generators():
    s = 42 + 128
    want = []
    for _ in range(32):
        s = (s * 6364136223846793005 + 1) & 0xFFFFFFFFFFFFFFFF
        f = np.float32(np.float32(((s >> 33) & 0xFFFFFFFF) % 200) - np.float32(100.0)) * np.float32(0.01)
        want.append(int(np.array([f], np.float32).view(np.uint32)[0] >> 16))
    assert list(oracle.lcg_bf16(32, 42 + 128)) == want
    p = oracle.bf16_to_f32(oracle.periodic_bf16(40, 17, 8))
    assert abs(p[0] - (-0.08)) < 1e-3 and abs(p[17] - (-0.08)) < 1e-3 and abs(p[8]) == 0.0


def test_ce_known_answer():
    logits = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    t = np.array([2], np.uint32)
    loss = oracle.ce_loss_forward(logits, t)
    assert abs(loss[0] - 1.44019) < 1e-3
    d = oracle.ce_loss_backward(logits, t, 1.0)
    assert abs(d.sum()) < 1e-6
    probs = oracle.softmax_forward(logits)
    assert abs(oracle.ce_mean_loss_from_probs(probs, t) - 1.44019) < 1e-3


def test_softmax_known_answers():
    x = np.arange(1, 9, dtype=np.float32).reshape(2, 4)
    y = oracle.softmax_forward(x)
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-6)
    y1 = oracle.softmax_forward(x[:1])
    dx = oracle.softmax_backward(np.array([[1, 0, 0, 0]], np.float32), y1)
    assert abs(dx.sum()) < 1e-6


def test_rmsnorm_known_answers():
    x = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    w = np.ones(4, np.float32)
    out, inv = oracle.rmsnorm_forward(x, w, 1e-5)
    rms = np.sqrt(np.float32(7.5) + np.float32(1e-5))
    assert np.allclose(out, x / rms, atol=1e-5)
    dx = oracle.rmsnorm_backward(np.array([[1, 0, 0, 0]], np.float32), x, w, 1e-5)
    assert abs(float((dx * x).sum())) < 1e-4
    # Ignis test: [[1,2],[3,4]] -> 0.6325, 1.2649 in row 0
    out2, _ = oracle.rmsnorm_forward(np.array([[1, 2], [3, 4]], np.float32), np.ones(2, np.float32), 1e-5)
    assert abs(out2[0, 0] - 0.6325) < 1e-3 and abs(out2[0, 1] - 1.2649) < 1e-3
    # dgamma against a float64 formulation
    rng = np.random.default_rng(3)
    xx = rng.standard_normal((9, 33)).astype(np.float32)
    dy = rng.standard_normal((9, 33)).astype(np.float32)
    r = 1.0 / np.sqrt((xx.astype(np.float64) ** 2).mean(axis=1) + 1e-6)
    want = (dy * xx * r[:, None]).sum(axis=0)
    assert np.allclose(oracle.rmsnorm_dgamma(dy, xx, 1e-6), want, rtol=1e-4, atol=1e-5)


def test_silu_and_adamw_against_float64():
    rng = np.random.default_rng(5)
    g = rng.standard_normal(257).astype(np.float32)
    u = rng.standard_normal(257).astype(np.float32)
    gr = rng.standard_normal(257).astype(np.float32)
    sig = 1 / (1 + np.exp(-g.astype(np.float64)))
    assert np.allclose(oracle.silu_gate_forward(g, u), g * sig * u, rtol=1e-5, atol=1e-6)
    dgate, dup = oracle.silu_gate_backward(gr, g, u)
    assert np.allclose(dup, gr * g * sig, rtol=1e-5, atol=1e-6)
    assert np.allclose(dgate, gr * u * sig * (1 + g * (1 - sig)), rtol=1e-5, atol=1e-6)
    p = rng.standard_normal(100).astype(np.float32)
    grad = rng.standard_normal(100).astype(np.float32)
    p2, m2, v2 = oracle.adamw_step(p, grad, np.zeros(100, np.float32), np.zeros(100, np.float32),
                                   1e-3, 0.9, 0.999, 1e-8, 0.01, 1)
    # step 1: m_hat = grad, v_hat = grad^2 -> update = lr * sign(grad) (approximately)
    want = p * (1 - 1e-3 * 0.01) - 1e-3 * grad / (np.abs(grad) + 1e-8)
    assert np.allclose(p2, want, rtol=1e-4, atol=1e-6)


def test_embedding_known_answers():
    """src/t0/embedding_kernels.rs:137-165: the reference's two CPU known-answer tests."""
    table = np.arange(1, 10, dtype=np.float32).reshape(3, 3)
    out = oracle.embedding_forward(table, [2, 0, 1], 3)
    assert np.array_equal(out, np.array([[7, 8, 9], [1, 2, 3], [4, 5, 6]], np.float32))
    grad_out = np.array([[1, 1, 1], [2, 2, 2], [3, 3, 3]], np.float32)
    gt = oracle.embedding_backward(np.zeros((2, 3), np.float32), [1, 0, 1], grad_out, 3)
    assert np.array_equal(gt, np.array([[2, 2, 2], [4, 4, 4]], np.float32))      # row 0 = token 1, row 1 = tokens 0 + 2
