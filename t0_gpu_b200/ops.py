"""Host-side mirror of the Ignis ops on the GEMM path (src/ignis/ops/bf16_matmul.rs, rmsnorm.rs,
cross_entropy.rs, silu.rs): f32 device buffers in and out, bf16 multiplicands, f32 accumulation.

Where the reference converts f32 -> bf16 and transposes on the host through the VRAM mapping
(bf16_matmul.rs:357-424), these functions run the cast kernel on the device and select the operand layout with
the GEMM's transpose flags, so no operand is ever transposed or padded.
"""
from __future__ import annotations

from typing import Optional, Tuple

from ._lib import lib
from .gpu_context import OUT_F32, GpuBuffer, GpuRuntime

RMSNORM_EPS = 1e-5   # the constant Ignis hard-codes (src/ignis/ops/rmsnorm.rs:18); pass eps explicitly to override


def _bf16_of(rt: GpuRuntime, buf: GpuBuffer, n: int) -> GpuBuffer:
    """A temporary bf16 copy of an activation (cast on the device, stream-ordered)."""
    out = rt.alloc(max(n * 2, 16))
    rt._check(lib().t0b_cast_f32_to_bf16(rt.handle, buf.gpu_addr(), out.gpu_addr(), n, 1))
    return out


def _weight_bf16(rt: GpuRuntime, w: GpuBuffer, n: int, weight_id: Optional[int]) -> GpuBuffer:
    """The cached bf16 copy of a weight (gpu_context.rs:392-432), keyed by `weight_id` or, without one, by the f32
    buffer's device address.  It is converted once and reused by every forward and backward call until
    `weight_updated` / `adamw_step` invalidates it."""
    return rt.get_or_create_bf16(weight_id if weight_id is not None else w.gpu_addr(), w, n)


def weight_updated(rt: GpuRuntime, w: GpuBuffer, weight_id: Optional[int] = None) -> None:
    """Tell the runtime that `w` changed (an optimizer step wrote it): its cached bf16 copy is dropped."""
    rt.invalidate_bf16(weight_id if weight_id is not None else w.gpu_addr())


# Every function below only queues work on the runtime's stream and returns (the reference waits for the queue to go
# idle after every op, src/ignis/ops/bf16_matmul.rs:162-207).  Results are complete once the caller reads them
# (`GpuBuffer.read` is ordered on the same stream) or calls `rt.synchronize()`.  Temporary buffers go back to the pool
# as soon as the launches that use them are queued: the pool hands them out again only to later work of the stream.

def dispatch_gemm_forward(rt: GpuRuntime, x: GpuBuffer, w: GpuBuffer, m: int, k: int, n: int,
                          weight_id: Optional[int] = None) -> GpuBuffer:
    """Y[M,N] f32 = X[M,K] f32 * W[K,N] f32 via bf16 (bf16_matmul.rs:162-207)."""
    x16, w16 = _bf16_of(rt, x, m * k), _weight_bf16(rt, w, k * n, weight_id)
    y = rt.alloc(max(m * n * 4, 16))
    rt.gemm(x16, w16, y, m, n, k, trans_a=False, trans_b=False, async_=True)
    rt.recycle(x16)
    return y


def gemm_backward_data(rt: GpuRuntime, dy: GpuBuffer, w: GpuBuffer, m: int, k: int, n: int,
                       weight_id: Optional[int] = None) -> GpuBuffer:
    """dX[M,K] = dY[M,N] * W[K,N]^T (bf16_matmul.rs:215-258): W is read as the [N_gemm, K_gemm] operand."""
    dy16, w16 = _bf16_of(rt, dy, m * n), _weight_bf16(rt, w, k * n, weight_id)
    dx = rt.alloc(max(m * k * 4, 16))
    rt.gemm(dy16, w16, dx, m, k, n, trans_a=False, trans_b=True, async_=True)
    rt.recycle(dy16)
    return dx


def gemm_backward_weight(rt: GpuRuntime, x: GpuBuffer, dy: GpuBuffer, m: int, k: int, n: int) -> GpuBuffer:
    """dW[K,N] = X[M,K]^T * dY[M,N] (bf16_matmul.rs:265-308): X is read transposed, no host transposes."""
    x16, dy16 = _bf16_of(rt, x, m * k), _bf16_of(rt, dy, m * n)
    dw = rt.alloc(max(k * n * 4, 16))
    rt.gemm(x16, dy16, dw, k, n, m, trans_a=True, trans_b=False, async_=True)
    rt.recycle(x16)
    rt.recycle(dy16)
    return dw


def matmul(rt: GpuRuntime, x: GpuBuffer, w: GpuBuffer, m: int, k: int, n: int, weight_id: Optional[int] = None):
    """`ops::bf16_matmul::matmul` (bf16_matmul.rs:33-98): returns (y, backward) where backward(dy) gives (dx, dw),
    the closure the reference records on its tape.  The bf16 copy of W is taken from the runtime's cache."""
    y = dispatch_gemm_forward(rt, x, w, m, k, n, weight_id)

    def backward(dy: GpuBuffer, x_needs: bool = True, w_needs: bool = True):
        dx = gemm_backward_data(rt, dy, w, m, k, n, weight_id) if x_needs else None
        dw = gemm_backward_weight(rt, x, dy, m, k, n) if w_needs else None
        return dx, dw

    return y, backward


def matmul_with_wt_bf16(rt: GpuRuntime, x: GpuBuffer, wt_bf16: GpuBuffer, m: int, k: int, n: int) -> GpuBuffer:
    """`ops::bf16_matmul::matmul_with_wt_bf16` (bf16_matmul.rs:102-134): Y[M,N] f32 = X[M,K] f32 (cast to bf16 on the
    device) times a weight already stored transposed as bf16 WT[N,K] -- the inference / repeated-forward form.
    No padding of M or N is needed."""
    x16 = _bf16_of(rt, x, m * k)
    y = rt.alloc(max(m * n * 4, 16))
    rt.gemm(x16, wt_bf16, y, m, n, k, trans_a=False, trans_b=True, async_=True)
    rt.recycle(x16)
    return y


def adamw_step(rt: GpuRuntime, param: GpuBuffer, grad: GpuBuffer, m_state: GpuBuffer, v_state: GpuBuffer, n: int, t: int,
               lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01,
               weight_id: Optional[int] = None) -> None:
    """One fused AdamW update of an f32 parameter buffer (src/t0/adamw_kernels.rs:35-119), after which the parameter's
    cached bf16 copy is invalidated, as the reference does after each optimizer step."""
    rt._check(lib().t0b_adamw_step(rt.handle, param.gpu_addr(), grad.gpu_addr(), m_state.gpu_addr(), v_state.gpu_addr(), 0, n,
                                   lr, beta1, beta2, eps, weight_decay, t, 1.0, 1))
    weight_updated(rt, param, weight_id)


def rmsnorm(rt: GpuRuntime, x: GpuBuffer, gamma: GpuBuffer, rows: int, dim: int, eps: float = RMSNORM_EPS):
    """`ops::rmsnorm::rmsnorm` (rmsnorm.rs:26-305): returns (y, backward) with backward(dy) -> (dx, dgamma)."""
    L = lib()
    y = rt.alloc(max(rows * dim * 4, 16))
    rt._check(L.t0b_rmsnorm_fwd(rt.handle, x.gpu_addr(), gamma.gpu_addr(), y.gpu_addr(), 0, rows, dim, eps, 0))

    def backward(dy: GpuBuffer) -> Tuple[GpuBuffer, GpuBuffer]:
        dx, dg = rt.alloc(max(rows * dim * 4, 16)), rt.alloc(max(dim * 4, 16))
        nbytes = L.t0b_rmsnorm_bwd_scratch_bytes(rows, dim)
        scratch = rt.alloc(nbytes)
        rt._check(L.t0b_rmsnorm_bwd(rt.handle, dy.gpu_addr(), x.gpu_addr(), gamma.gpu_addr(), dx.gpu_addr(), dg.gpu_addr(),
                                    scratch.gpu_addr(), nbytes, rows, dim, eps, 0))
        rt.recycle(scratch)
        return dx, dg

    return y, backward


def cross_entropy(rt: GpuRuntime, logits: GpuBuffer, targets: GpuBuffer, batch: int, cols: int):
    """`ops::cross_entropy::cross_entropy` (cross_entropy.rs:34-115): mean loss over the batch and
    grad = (softmax - onehot) / batch, both computed on the device (the reference reads the probabilities back
    and finishes on the CPU)."""
    import numpy as np

    L = lib()
    losses, grad = rt.alloc(max(batch * 4, 16)), rt.alloc(max(batch * cols * 4, 16))
    rt._check(L.t0b_softmax_ce(rt.handle, logits.gpu_addr(), targets.gpu_addr(), losses.gpu_addr(), grad.gpu_addr(), batch,
                               cols, cols, 1.0 / batch, 0))
    loss = float(losses.read_as(np.float32, batch).mean())
    rt.recycle(losses)
    return loss, grad


def embedding_forward(rt: GpuRuntime, table: GpuBuffer, ids: GpuBuffer, seq_len: int, dim: int, vocab_size: int):
    """`ops::embedding::embedding_forward(table, ids_buf, seq_len, dim, runtime)` (embedding.rs:25-178): gathers
    table rows; returns (out, backward) where backward(grad_out) -> grad_table, a zeroed [vocab, dim] buffer with the
    rows of grad_out added in token order (the reference's scatter uses unordered atomics)."""
    L = lib()
    out = rt.alloc(max(seq_len * dim * 4, 16))
    rt._check(L.t0b_embedding_fwd(rt.handle, table.gpu_addr(), ids.gpu_addr(), out.gpu_addr(), seq_len, dim, vocab_size, 0))

    def backward(grad_out: GpuBuffer) -> GpuBuffer:
        grad_table = rt.alloc_zero(max(vocab_size * dim * 4, 16))
        rt._check(L.t0b_embedding_bwd(rt.handle, grad_table.gpu_addr(), ids.gpu_addr(), grad_out.gpu_addr(), seq_len, dim,
                                      vocab_size, 0, 0, 0))
        return grad_table

    return out, backward
