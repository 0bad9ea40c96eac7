"""numpy-facing wrapper over the C oracle (oracle/t0_oracle.c).

TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the CPU-baseline leg of bench.py.
The product (t0_gpu_b200 and its CUDA library) never imports this package.

Parity status: pinned -- tests/test_oracle_golden.py checks these functions against the
reference's torch-generated golden vectors and closed-form known answers.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.OUT
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(_build.SRC):
            path = _build.build()
        _LIB = C.CDLL(path)
        _declare(_LIB)
    return _LIB


_P = C.c_void_p
_I64 = C.c_int64
_SZ = C.c_size_t


def _declare(L: C.CDLL) -> None:
    L.t0o_f32_to_bf16_rne.argtypes = [C.c_float]
    L.t0o_f32_to_bf16_rne.restype = C.c_uint16
    L.t0o_f32_to_bf16_trunc.argtypes = [C.c_float]
    L.t0o_f32_to_bf16_trunc.restype = C.c_uint16
    L.t0o_bf16_to_f32.argtypes = [C.c_uint16]
    L.t0o_bf16_to_f32.restype = C.c_float
    L.t0o_f32_to_bf16_rne_array.argtypes = [_P, _P, _SZ]
    L.t0o_bf16_to_f32_array.argtypes = [_P, _P, _SZ]
    L.t0o_rand_bf16.argtypes = [_P, _SZ, C.c_uint64]
    L.t0o_lcg_bf16.argtypes = [_P, _SZ, C.c_uint64]
    L.t0o_periodic_bf16.argtypes = [_P, _SZ, C.c_uint32, C.c_int32]
    L.t0o_gemm_bf16.argtypes = [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, C.c_int, C.c_int, _I64, _I64, C.c_int]
    L.t0o_splitk_reduce.argtypes = [_P, _P, _SZ, C.c_int]
    L.t0o_gemm_bf16_nt_krange.argtypes = [_P, _P, _P, _I64, _I64, _I64, _I64, _I64]
    L.t0o_transpose_bf16.argtypes = [_P, _P, _I64, _I64]
    L.t0o_epilogue_bias.argtypes = [_P, _P, _I64, _I64, _I64, C.c_int]
    L.t0o_rmsnorm_forward.argtypes = [_P, _P, _P, _P, _I64, _I64, C.c_float]
    L.t0o_rmsnorm_backward.argtypes = [_P, _P, _P, _P, _I64, _I64, C.c_float]
    L.t0o_rmsnorm_dgamma.argtypes = [_P, _P, _P, _I64, _I64, C.c_float]
    L.t0o_softmax_forward.argtypes = [_P, _P, _I64, _I64]
    L.t0o_softmax_backward.argtypes = [_P, _P, _P, _I64, _I64]
    L.t0o_ce_loss_forward.argtypes = [_P, _P, _P, _I64, _I64]
    L.t0o_ce_loss_backward.argtypes = [_P, _P, _P, _I64, _I64, C.c_float]
    L.t0o_ce_mean_loss_from_probs.argtypes = [_P, _P, _I64, _I64]
    L.t0o_ce_mean_loss_from_probs.restype = C.c_float
    L.t0o_silu_gate_forward.argtypes = [_P, _P, _P, _SZ]
    L.t0o_silu_gate_backward.argtypes = [_P, _P, _P, _P, _P, _SZ]
    L.t0o_residual_add.argtypes = [_P, _P, _SZ]
    L.t0o_embedding_forward.argtypes = [_P, _P, _P, _SZ, _SZ]
    L.t0o_embedding_backward.argtypes = [_P, _P, _P, _SZ, _SZ]
    L.t0o_adamw_step.argtypes = [_P, _P, _P, _P, _SZ, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_uint32]


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"], "oracle wants contiguous arrays"
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u16(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint16)


# ---------------------------------------------------------------------------------------------- bf16

def f32_to_bf16_rne(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().t0o_f32_to_bf16_rne_array(_ptr(x), _ptr(out), x.size)
    return out


def f32_to_bf16_trunc(x) -> np.ndarray:
    return (_f32(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_to_f32(x) -> np.ndarray:
    x = _u16(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().t0o_bf16_to_f32_array(_ptr(x), _ptr(out), x.size)
    return out


# ---------------------------------------------------------------------------------------------- generators

def rand_bf16(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().t0o_rand_bf16(_ptr(out), n, C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF))
    return out


def lcg_bf16(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().t0o_lcg_bf16(_ptr(out), n, C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF))
    return out


def periodic_bf16(n: int, period: int, offset: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    lib().t0o_periodic_bf16(_ptr(out), n, period, offset)
    return out


def normal_bf16(shape, seed: int, scale: float) -> np.ndarray:
    """N(0,1) * scale rounded (RNE) to bf16 bit patterns; numpy Philox stream keyed by seed.

    The benchmark configs ask for N(0,1)/sqrt(K) inputs; the reference itself has no normal
    generator, so this one is defined here and used by both sides of every comparison."""
    rng = np.random.Generator(np.random.Philox(seed))
    x = rng.standard_normal(size=shape, dtype=np.float32) * np.float32(scale)
    return f32_to_bf16_rne(x)


# ---------------------------------------------------------------------------------------------- GEMM

def gemm_bf16(a, b, m: int, n: int, k: int, trans_a: bool = False, trans_b: bool = True,
              lda: int | None = None, ldb: int | None = None, threads: int = 1,
              row_begin: int = 0, row_end: int | None = None) -> np.ndarray:
    """C[M,N] f32 = op(A) * op(B), bf16 bit-pattern inputs, k-ascending unfused f32 accumulate.

    trans_a False: A stored [M,K]; True: A stored [K,M].
    trans_b True : B stored [N,K] (the reference's NT default); False: B stored [K,N].
    Only rows [row_begin, row_end) of C are computed (others left at zero)."""
    a = _u16(a)
    b = _u16(b)
    if lda is None:
        lda = m if trans_a else k
    if ldb is None:
        ldb = k if trans_b else n
    if row_end is None:
        row_end = m
    c = np.zeros((m, n), dtype=np.float32)
    lib().t0o_gemm_bf16(_ptr(a), _ptr(b), _ptr(c), m, n, k, lda, ldb, n, int(trans_a), int(trans_b),
                        row_begin, row_end, threads)
    return c


def gemm_nt_krange(x, wt, m: int, n: int, k: int, k_begin: int, k_end: int) -> np.ndarray:
    x = _u16(x)
    wt = _u16(wt)
    y = np.zeros((m, n), dtype=np.float32)
    lib().t0o_gemm_bf16_nt_krange(_ptr(x), _ptr(wt), _ptr(y), m, n, k, k_begin, k_end)
    return y


def splitk_reduce(partials, sk: int) -> np.ndarray:
    partials = _f32(partials)
    total = partials.size // sk
    y = np.empty(total, dtype=np.float32)
    lib().t0o_splitk_reduce(_ptr(partials), _ptr(y), total, sk)
    return y


def transpose_bf16(a, rows: int, cols: int) -> np.ndarray:
    a = _u16(a)
    out = np.empty(rows * cols, dtype=np.uint16)
    lib().t0o_transpose_bf16(_ptr(a), _ptr(out), rows, cols)
    return out


def epilogue_bias(y, bias, relu: bool) -> np.ndarray:
    y = _f32(y).copy()
    bias = _f32(bias)
    m, n = y.shape
    lib().t0o_epilogue_bias(_ptr(y), _ptr(bias), m, n, n, int(relu))
    return y


# ---------------------------------------------------------------------------------------------- norm / softmax / CE

def rmsnorm_forward(x, weight, eps: float):
    x = _f32(x)
    weight = _f32(weight)
    rows, cols = x.shape
    out = np.empty_like(x)
    inv = np.empty(rows, dtype=np.float32)
    lib().t0o_rmsnorm_forward(_ptr(x), _ptr(weight), _ptr(out), _ptr(inv), rows, cols, eps)
    return out, inv


def rmsnorm_backward(dy, x, weight, eps: float) -> np.ndarray:
    dy = _f32(dy)
    x = _f32(x)
    weight = _f32(weight)
    rows, cols = x.shape
    dx = np.empty_like(x)
    lib().t0o_rmsnorm_backward(_ptr(dy), _ptr(x), _ptr(weight), _ptr(dx), rows, cols, eps)
    return dx


def rmsnorm_dgamma(dy, x, eps: float) -> np.ndarray:
    dy = _f32(dy)
    x = _f32(x)
    rows, cols = x.shape
    dg = np.empty(cols, dtype=np.float32)
    lib().t0o_rmsnorm_dgamma(_ptr(dy), _ptr(x), _ptr(dg), rows, cols, eps)
    return dg


def softmax_forward(x) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    lib().t0o_softmax_forward(_ptr(x), _ptr(out), rows, cols)
    return out


def softmax_backward(dy, y) -> np.ndarray:
    dy = _f32(dy)
    y = _f32(y)
    rows, cols = y.shape
    dx = np.empty_like(y)
    lib().t0o_softmax_backward(_ptr(dy), _ptr(y), _ptr(dx), rows, cols)
    return dx


def ce_loss_forward(logits, targets) -> np.ndarray:
    logits = _f32(logits)
    targets = np.ascontiguousarray(targets, dtype=np.uint32)
    rows, cols = logits.shape
    losses = np.empty(rows, dtype=np.float32)
    lib().t0o_ce_loss_forward(_ptr(logits), _ptr(targets), _ptr(losses), rows, cols)
    return losses


def ce_loss_backward(logits, targets, scale: float) -> np.ndarray:
    logits = _f32(logits)
    targets = np.ascontiguousarray(targets, dtype=np.uint32)
    rows, cols = logits.shape
    d = np.empty_like(logits)
    lib().t0o_ce_loss_backward(_ptr(logits), _ptr(targets), _ptr(d), rows, cols, scale)
    return d


def ce_mean_loss_from_probs(probs, targets) -> float:
    probs = _f32(probs)
    targets = np.ascontiguousarray(targets, dtype=np.uint32)
    rows, cols = probs.shape
    return float(lib().t0o_ce_mean_loss_from_probs(_ptr(probs), _ptr(targets), rows, cols))


# ---------------------------------------------------------------------------------------------- elementwise

def silu_gate_forward(gate, up) -> np.ndarray:
    gate = _f32(gate)
    up = _f32(up)
    out = np.empty_like(gate)
    lib().t0o_silu_gate_forward(_ptr(gate), _ptr(up), _ptr(out), gate.size)
    return out


def silu_gate_backward(grad, gate, up):
    grad = _f32(grad)
    gate = _f32(gate)
    up = _f32(up)
    dgate = np.empty_like(gate)
    dup = np.empty_like(gate)
    lib().t0o_silu_gate_backward(_ptr(grad), _ptr(gate), _ptr(up), _ptr(dgate), _ptr(dup), gate.size)
    return dgate, dup


def residual_add(y, x) -> np.ndarray:
    y = _f32(y).copy()
    x = _f32(x)
    lib().t0o_residual_add(_ptr(y), _ptr(x), y.size)
    return y


def embedding_forward(table, indices, dim: int) -> np.ndarray:
    table = _f32(table)
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    out = np.empty((idx.size, dim), np.float32)
    lib().t0o_embedding_forward(_ptr(table), _ptr(idx), _ptr(out), idx.size, dim)
    return out


def embedding_backward(grad_table, indices, grad_output, dim: int) -> np.ndarray:
    """Returns grad_table + the scattered rows of grad_output (tokens added in ascending order)."""
    gt = _f32(grad_table).copy()
    idx = np.ascontiguousarray(indices, dtype=np.uint32)
    go = _f32(grad_output)
    lib().t0o_embedding_backward(_ptr(gt), _ptr(idx), _ptr(go), idx.size, dim)
    return gt


def adamw_step(params, grads, m, v, lr, beta1, beta2, eps, weight_decay, t):
    params = _f32(params).copy()
    grads = _f32(grads)
    m = _f32(m).copy()
    v = _f32(v).copy()
    lib().t0o_adamw_step(_ptr(params), _ptr(grads), _ptr(m), _ptr(v), params.size, lr, beta1, beta2, eps,
                         weight_decay, t)
    return params, m, v
