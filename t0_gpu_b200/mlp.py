"""The Ignis MLP training step on the B200 kernels, data-parallel over the GPUs of one node.

Model (the benchmark's fifth config): input 4096 -> 3 x [Linear(4096) -> RMSNorm(eps 1e-6, weight 1) -> SiLU] ->
Linear(32000) -> softmax cross-entropy.  bf16 compute copies of fp32 master weights (Kaiming-uniform), f32
activations between kernels, bf16 operands into every GEMM, f32 accumulation, f32 gradients.

The step follows the structure of the reference's training loop (examples/train_mlp.rs:121-233: forward, loss,
backward, AdamW) with the ops of the hot path: `matmul` forward / backward-data / backward-weight
(src/ignis/ops/bf16_matmul.rs:33-308) without its host-side conversions and transposes, `rmsnorm`
(src/ignis/ops/rmsnorm.rs:26-305), SiLU (src/ignis/ops/silu.rs:32-152), `cross_entropy`
(src/ignis/ops/cross_entropy.rs:34-115) with loss and gradient computed on the device, AdamW
(src/t0/adamw_kernels.rs:35-119).  Data parallelism (rows split over ranks, fp32 gradient all-reduce) has no
counterpart in the reference; `torch.distributed` carries the all-reduce, started per layer as soon as that
layer's weight gradient is ready so it overlaps the rest of the backward pass.  With `shard_optimizer=True` the
gradients are reduce-scattered instead, every rank runs AdamW on its 1/world slice of each tensor and the updated
copies are all-gathered: half the gradient bytes on NVLink and 1/world of the optimizer's HBM traffic per rank, the
same update per element.

Device memory comes from torch tensors (the all-reduce needs them); every kernel is a C-ABI call.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import os

from ._lib import lib
from .gpu_context import OUT_BF16, OUT_F32, GpuRuntime


def _nvtx_push(name: str) -> None:
    """Open an NVTX range around a phase of the step when T0B_NVTX=1 (forward, loss, backward with its gradient
    exchange, the optimizer), for a timeline profiler; otherwise nothing."""
    if os.environ.get("T0B_NVTX", "0") == "1":
        import torch

        torch.cuda.nvtx.range_push(name)


def _nvtx_pop() -> None:
    if os.environ.get("T0B_NVTX", "0") == "1":
        import torch

        torch.cuda.nvtx.range_pop()



@dataclass
class MlpConfig:
    d_in: int = 4096
    hidden: List[int] = field(default_factory=lambda: [4096, 4096, 4096])
    n_classes: int = 32000
    eps: float = 1e-6
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    adam_eps: float = 1e-8
    weight_decay: float = 0.01

    def dims(self):
        d = [self.d_in] + list(self.hidden) + [self.n_classes]
        return list(zip(d[:-1], d[1:]))          # (fan_in, fan_out) per Linear

    def flops_per_row(self) -> float:
        """Forward + backward GEMM FLOPs per batch row (2 MNK each; dX is not needed for the first layer)."""
        f = 0.0
        for i, (k, n) in enumerate(self.dims()):
            f += 2.0 * k * n * (2 if i == 0 else 3)
        return f


def kaiming_uniform_(torch, w, fan_in: int, seed: int):
    """U(-sqrt(6 / fan_in), +sqrt(6 / fan_in)), seeded per tensor."""
    g = torch.Generator(device=w.device)
    g.manual_seed(seed)
    bound = (6.0 / fan_in) ** 0.5
    w.uniform_(-bound, bound, generator=g)
    return w


def exchange_units(dims, hidden, want_shard: bool, out_panels: int = 4):
    """Units of the data-parallel gradient exchange over the flat parameter buffer (weights layer by layer, then all
    gammas): a list of (offset, numel), the unit ids of every layer, and the id of the gamma unit.  One unit per weight
    matrix; the output layer's (by far the largest) is cut into `out_panels` row panels when the optimizer is sharded,
    so that its exchange starts after the first panel's GEMM instead of after the whole gradient; one unit for all
    gammas together."""
    units, layer_units, off = [], [], 0
    nl = len(dims)
    for i, (k_i, n_i) in enumerate(dims):
        panels = out_panels if (want_shard and i == nl - 1 and k_i % out_panels == 0) else 1
        per = k_i // panels
        ids = []
        for pnl in range(panels):
            ids.append(len(units))
            units.append((off + pnl * per * n_i, per * n_i))
        layer_units.append(ids)
        off += k_i * n_i
    gamma_unit = len(units)
    units.append((off, sum(hidden)))
    return units, layer_units, gamma_unit


def shard_range(unit, rank: int, world: int):
    """[lo, hi) of the slice of `unit` = (offset, numel) that `rank` owns under the sharded optimizer."""
    off, n = unit
    ns = n // world
    return off + rank * ns, off + (rank + 1) * ns


class MlpTrainer:
    """One data-parallel replica.  `rows` is this rank's share of the batch, `rows_total` the global batch."""

    def __init__(self, rt: GpuRuntime, cfg: MlpConfig, rows: int, rows_total: Optional[int] = None, group=None,
                 seed: int = 100, shard_optimizer: bool = False, autotune: bool = True, local_only: bool = False):
        """local_only: a single-rank replica even while a process group is up (no gradient exchange) -- the one-rank
        side of a data-parallel equivalence check."""
        import torch
        import torch.distributed as dist

        self.torch, self.rt, self.cfg, self.rows, self.group = torch, rt, cfg, rows, group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and not local_only) else 1
        self.rows_total = rows_total if rows_total is not None else rows * self.world
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.L = lib()
        # The library's launches and torch's own work (fills, all-reduce hand-off) share one non-default stream.
        if torch.cuda.current_stream().cuda_stream == 0:
            self.stream = torch.cuda.Stream(device=self.dev)
            torch.cuda.set_stream(self.stream)
        else:
            self.stream = torch.cuda.current_stream()
        rt.set_stream(self.stream.cuda_stream)
        # With several ranks the collectives run beside the persistent GEMMs.  T0B_COMM_SMS=n keeps n SMs out of the
        # GEMMs' grids for them; measured on two GPUs it does not pay (step 2.53 ms with 0, 2.55-2.62 ms with 8-32),
        # so the default is 0.
        if self.world > 1:
            import os
            spare = int(os.environ.get("T0B_COMM_SMS", "0"))
            if spare > 0:
                rt.set_sm_limit(max(2, rt.num_sms() - spare))
        dims = cfg.dims()
        f32, bf16 = torch.float32, torch.bfloat16
        # Parameters: W_l stored [fan_in, fan_out] (row-major [K, N], the layout `Linear` uses), gamma_l = 1.
        sizes = [k * n for k, n in dims] + list(cfg.hidden)
        self.n_params = sum(sizes)
        self.master = torch.empty(self.n_params, dtype=f32, device=self.dev)
        self.grads = torch.zeros(self.n_params, dtype=f32, device=self.dev)
        self.compute = torch.empty(self.n_params, dtype=bf16, device=self.dev)   # bf16 copies (gammas unused)
        offs, o = [], 0
        for s in sizes:
            offs.append(o)
            o += s
        nl = len(dims)
        want_shard = bool(shard_optimizer) and self.world > 1
        self._units, self._layer_units, self._gamma_unit = exchange_units(dims, cfg.hidden, want_shard)
        # Sharded optimizer (more than one rank): every unit's gradient is reduce-scattered instead of all-reduced, each
        # rank keeps AdamW state for, and updates, its 1/world slice of every unit, and the updated bf16 copies (f32
        # for the gammas) are all-gathered.  Per rank this moves half the gradient bytes over NVLink, a 1/world share
        # of the AdamW traffic through HBM, and the same arithmetic per element as the replicated update.
        self.sharded = want_shard and all(n % self.world == 0 for _, n in self._units)
        if self.sharded:
            self.rank = dist.get_rank(group)
            self.grad_shards = [torch.empty(n // self.world, dtype=f32, device=self.dev) for _, n in self._units]
            self.m_shards = [torch.zeros(n // self.world, dtype=f32, device=self.dev) for _, n in self._units]
            self.v_shards = [torch.zeros(n // self.world, dtype=f32, device=self.dev) for _, n in self._units]
        else:
            self.adam_m = torch.zeros(self.n_params, dtype=f32, device=self.dev)
            self.adam_v = torch.zeros(self.n_params, dtype=f32, device=self.dev)
        self.w = [self.master[offs[i]:offs[i] + sizes[i]].view(dims[i]) for i in range(nl)]
        self.w16 = [self.compute[offs[i]:offs[i] + sizes[i]].view(dims[i]) for i in range(nl)]
        self.dw = [self.grads[offs[i]:offs[i] + sizes[i]].view(dims[i]) for i in range(nl)]
        self.gamma = [self.master[offs[nl + i]:offs[nl + i] + sizes[nl + i]] for i in range(len(cfg.hidden))]
        self.dgamma = [self.grads[offs[nl + i]:offs[nl + i] + sizes[nl + i]] for i in range(len(cfg.hidden))]
        for i, (k, n) in enumerate(dims):
            kaiming_uniform_(torch, self.w[i], k, seed + i)
        for g in self.gamma:
            g.fill_(1.0)
        self._refresh_compute_copies()
        # Activations.
        B = rows
        self.x16 = torch.empty((B, cfg.d_in), dtype=bf16, device=self.dev)
        self.z = [torch.empty((B, h), dtype=f32, device=self.dev) for h in cfg.hidden]        # Linear outputs
        self.h16 = [torch.empty((B, h), dtype=bf16, device=self.dev) for h in cfg.hidden]     # bf16 layer outputs
        self.logits = torch.empty((B, cfg.n_classes), dtype=f32, device=self.dev)
        self.dlogits16 = torch.empty((B, cfg.n_classes), dtype=bf16, device=self.dev)
        self.losses = torch.empty(B, dtype=f32, device=self.dev)
        self.dh = torch.empty((B, max(cfg.hidden)), dtype=f32, device=self.dev)
        self.dz16 = torch.empty((B, max(cfg.hidden)), dtype=bf16, device=self.dev)
        self.scratch_bytes = self.L.t0b_rmsnorm_bwd_scratch_bytes(B, max(cfg.hidden))
        self.scratch = torch.empty(self.scratch_bytes, dtype=torch.uint8, device=self.dev)
        self.step_count = 0
        self._pending = []
        self._updates = {}
        if autotune:
            self._tune_gemms()

    def _tune_gemms(self):
        """Measure the tile candidates for every GEMM shape of the step once (the reference's `auto_gemm` does the same
        on first use, src/t0/auto_gemm.rs:445-480); config-less GEMM calls of these shapes then use the winners."""
        cfg, B = self.cfg, self.rows
        shapes = set()
        k = cfg.d_in
        for n in cfg.hidden:
            shapes.add((B, n, k, False, False))          # forward
            shapes.add((k, n, B, True, False))           # dW
            shapes.add((B, k, n, False, True))           # dX
            k = n
        V = cfg.n_classes
        shapes.add((B, V, k, False, False))
        shapes.add((k // len(self._layer_units[-1]), V, B, True, False))
        shapes.add((B, k, V, False, True))
        done = self.rt.__dict__.setdefault("_mlp_tuned_shapes", set())   # a second trainer on this runtime measures nothing twice
        for shape in sorted(shapes - done):
            m, n, kk, ta, tb = shape
            self.rt.tune(m, n, kk, trans_a=ta, trans_b=tb)
            done.add(shape)

    # ------------------------------------------------------------------ helpers (each one C-ABI call)
    def _ck(self, rc):
        self.rt._check(rc)

    def _gemm(self, a, b, c, m, n, k, trans_a, trans_b, lda, ldb, out_dtype=OUT_F32):
        self._ck(self.L.t0b_gemm(self.rt.handle, None, int(trans_a), int(trans_b), a.data_ptr(), b.data_ptr(),
                                 c.data_ptr(), m, n, k, lda, ldb, n, out_dtype, 0, 0, 1.0, 0, 0, 1))

    def _cast(self, src, dst, n):
        self._ck(self.L.t0b_cast_f32_to_bf16(self.rt.handle, src.data_ptr(), dst.data_ptr(), n, 1))

    def _refresh_compute_copies(self):
        self._ck(self.L.t0b_cast_f32_to_bf16(self.rt.handle, self.master.data_ptr(), self.compute.data_ptr(),
                                             self.n_params, 1))

    # ------------------------------------------------------------------ one step
    def forward_backward(self, x, targets):
        """x: f32 [rows, d_in]; targets: int32/uint32 [rows].  Leaves the mean loss contribution of this rank in
        `self.losses` (per-row losses) and the summed-over-ranks gradients in `self.grads`."""
        cfg, B, L, h = self.cfg, self.rows, self.L, self.rt.handle
        nh = len(cfg.hidden)
        scale = 1.0 / float(self.rows_total)
        # forward
        _nvtx_push("t0b.mlp.forward")
        self._cast(x, self.x16, B * cfg.d_in)
        inp, k = self.x16, cfg.d_in
        self._wait_update(self._gamma_unit)      # gammas (read by every RMSNorm)
        for l in range(nh):
            n = cfg.hidden[l]
            self._wait_layer(l)
            self._gemm(inp, self.w16[l], self.z[l], B, n, k, False, False, k, n)
            # RMSNorm, SiLU and the bf16 down-cast in one pass over z (the f32 intermediates never reach memory)
            self._ck(L.t0b_rmsnorm_silu_fwd(h, self.z[l].data_ptr(), self.gamma[l].data_ptr(), self.h16[l].data_ptr(), 0, B, n,
                                            cfg.eps, 1))
            inp, k = self.h16[l], n
        V = cfg.n_classes
        self._wait_layer(nh)
        self._gemm(inp, self.w16[nh], self.logits, B, V, k, False, False, k, V)
        _nvtx_pop()
        # loss and its gradient, stored directly as the bf16 operand of the two GEMMs that follow
        _nvtx_push("t0b.mlp.loss")
        self._ck(L.t0b_softmax_ce_bf16(h, self.logits.data_ptr(), targets.data_ptr(), self.losses.data_ptr(),
                                       self.dlogits16.data_ptr(), B, V, V, scale, 1))
        _nvtx_pop()
        # backward
        _nvtx_push("t0b.mlp.backward")
        # dW_out[k, V] = h_last^T [k, B] * dlogits [B, V]: A stored [B, k] read transposed
        ids = self._layer_units[nh]
        per = k // len(ids)                     # rows of dW_out per panel = columns of h_last
        for pnl, u in enumerate(ids):
            self._gemm(inp[:, pnl * per:], self.dlogits16, self.dw[nh][pnl * per:], per, V, B, True, False, k, V)
            self._start_reduce(u)
        # dh_last[B, k] = dlogits [B, V] * W_out^T: B operand stored [k, V] = [N_gemm, K_gemm]
        self._gemm(self.dlogits16, self.w16[nh], self.dh, B, k, V, False, True, V, V)
        for l in range(nh - 1, -1, -1):
            n = cfg.hidden[l]
            k = cfg.hidden[l - 1] if l > 0 else cfg.d_in
            prev = self.h16[l - 1] if l > 0 else self.x16
            # SiLU backward on the recomputed RMSNorm output, RMSNorm backward and the bf16 down-cast in one pass
            self._ck(L.t0b_rmsnorm_silu_bwd(h, self.dh.data_ptr(), self.z[l].data_ptr(), self.gamma[l].data_ptr(),
                                            self.dz16.data_ptr(), self.dgamma[l].data_ptr(), self.scratch.data_ptr(),
                                            self.scratch_bytes, B, n, cfg.eps, 1))
            self._gemm(prev, self.dz16, self.dw[l], k, n, B, True, False, k, n)
            self._start_reduce(self._layer_units[l][0])
            if l > 0:
                self._gemm(self.dz16, self.w16[l], self.dh, B, k, n, False, True, n, n)
        if self.world > 1:
            self._start_reduce(self._gamma_unit) # the small gamma gradients go last, in one piece
        _nvtx_pop()
        _nvtx_push("t0b.mlp.grad_exchange_wait")
        self._finish_reduce()
        _nvtx_pop()

    def _start_reduce(self, unit: int):
        """Start the exchange of one unit's gradient: all-reduce (replicated optimizer) or reduce-scatter (sharded)."""
        if self.world == 1:
            return
        import torch.distributed as dist

        off, n = self._units[unit]
        flat = self.grads[off:off + n]
        if self.sharded:
            w = dist.reduce_scatter_tensor(self.grad_shards[unit], flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        else:
            w = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self._pending.append(w)

    def _finish_reduce(self):
        for w in self._pending:
            w.wait()
        self._pending = []

    def optimizer_step(self):
        cfg = self.cfg
        self.step_count += 1
        if not self.sharded:
            self._ck(self.L.t0b_adamw_step(self.rt.handle, self.master.data_ptr(), self.grads.data_ptr(),
                                           self.adam_m.data_ptr(), self.adam_v.data_ptr(), self.compute.data_ptr(),
                                           self.n_params, cfg.lr, cfg.beta1, cfg.beta2, cfg.adam_eps, cfg.weight_decay,
                                           self.step_count, 1.0, 1))
            return
        import torch.distributed as dist

        gamma_unit = self._gamma_unit
        # Units are updated and gathered in the order the next forward pass needs them (gammas, then the layers); the
        # forward pass waits for a unit right before its first use, so the gathers of the later (larger) layers run
        # behind the GEMMs of the earlier ones.
        for u in [gamma_unit] + list(range(gamma_unit)):   # unit ids follow the layer order
            off, n = self._units[u]
            lo, hi = shard_range(self._units[u], self.rank, self.world)
            ns = hi - lo
            own_master, own_bf16 = self.master[lo:hi], self.compute[lo:hi]
            self._ck(self.L.t0b_adamw_step(self.rt.handle, own_master.data_ptr(), self.grad_shards[u].data_ptr(),
                                           self.m_shards[u].data_ptr(), self.v_shards[u].data_ptr(), own_bf16.data_ptr(), ns,
                                           cfg.lr, cfg.beta1, cfg.beta2, cfg.adam_eps, cfg.weight_decay, self.step_count, 1.0, 1))
            # Every rank's slice sits at its own offset of the full buffer, so the gather is in place.  The GEMMs read
            # the bf16 copies; RMSNorm reads the f32 gammas, so that unit is gathered in f32.
            if u == gamma_unit:
                self._updates[u] = dist.all_gather_into_tensor(self.master[off:off + n], own_master, group=self.group, async_op=True)
            else:
                self._updates[u] = dist.all_gather_into_tensor(self.compute[off:off + n], own_bf16, group=self.group, async_op=True)

    def _wait_update(self, unit: int):
        """Make the stream wait for the all-gather that delivers `unit`'s updated parameters (sharded optimizer)."""
        w = self._updates.pop(unit, None)
        if w is not None:
            w.wait()

    def _wait_layer(self, layer: int):
        for u in self._layer_units[layer]:
            self._wait_update(u)

    def finish_updates(self):
        """Wait for every outstanding parameter gather (before reading `compute` or the gammas from outside a step)."""
        for u in list(self._updates):
            self._wait_update(u)

    def gather_master(self):
        """The full f32 master parameters (sharded optimizer: assembled from every rank's slices)."""
        if not self.sharded:
            return self.master.clone()
        import torch.distributed as dist

        self.finish_updates()
        out = self.master.clone()
        for unit in self._units:
            off, n = unit
            lo, hi = shard_range(unit, self.rank, self.world)
            dist.all_gather_into_tensor(out[off:off + n], self.master[lo:hi].clone(), group=self.group)
        return out

    def step(self, x, targets):
        self.forward_backward(x, targets)
        _nvtx_push("t0b.mlp.optimizer")
        self.optimizer_step()
        _nvtx_pop()

    def mean_loss(self) -> float:
        """Global mean loss: sum of this rank's per-row losses / rows_total, summed over ranks."""
        torch = self.torch
        s = self.losses.sum() / float(self.rows_total)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(s, group=self.group)
        return float(s.item())
