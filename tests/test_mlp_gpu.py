"""The MLP training step (Linear -> RMSNorm -> SiLU x3 -> Linear -> softmax cross-entropy) against a CPU
composition of the oracle's functions with casts at the same points: loss and every gradient, on a reduced-size
replica (GEMM tolerances for the weight gradients, 1e-3 relative for the loss), and data-parallel equivalence
(2 ranks x B/2 rows == 1 rank x B rows) when two GPUs are present."""
import os
import socket

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def oracle_step(x, targets, w16, gammas, eps, scale):
    """w16: list of bf16-bit arrays [k, n]; returns loss rows, dW list, dgamma list.

    The oracle reads B either as [K, N] or as [N, K]; the element order of every sum is the same (k ascending), so the
    forward products use a transposed copy of W, whose rows are contiguous for the oracle's inner loop."""
    B = x.shape[0]
    nh = len(gammas)
    wt16 = [np.ascontiguousarray(w.T) for w in w16]
    inp = oracle.f32_to_bf16_rne(x)
    zs, rs, hs = [], [], [inp]
    for l in range(nh):
        k, n = w16[l].shape
        z = oracle.gemm_bf16(inp, wt16[l], B, n, k, trans_a=False, trans_b=True, threads=8)
        r, _ = oracle.rmsnorm_forward(z, gammas[l], eps)
        a = oracle.silu_gate_forward(r, np.ones_like(r))
        inp = oracle.f32_to_bf16_rne(a)
        zs.append(z); rs.append(r); hs.append(inp)
    k, V = w16[nh].shape
    logits = oracle.gemm_bf16(inp, wt16[nh], B, V, k, trans_a=False, trans_b=True, threads=8)
    loss = oracle.ce_loss_forward(logits, targets)
    dl16 = oracle.f32_to_bf16_rne(oracle.ce_loss_backward(logits, targets, scale))
    dws = [None] * (nh + 1)
    dgs = [None] * nh
    dws[nh] = oracle.gemm_bf16(hs[nh], dl16, k, V, B, trans_a=True, trans_b=False, threads=8)
    dh = oracle.gemm_bf16(dl16, w16[nh], B, k, V, trans_a=False, trans_b=True, threads=8)
    for l in range(nh - 1, -1, -1):
        k, n = w16[l].shape
        dr, _ = oracle.silu_gate_backward(dh, rs[l], np.ones_like(rs[l]))
        dz = oracle.rmsnorm_backward(dr, zs[l], gammas[l], eps)
        dgs[l] = oracle.rmsnorm_dgamma(dr, zs[l], eps)
        dz16 = oracle.f32_to_bf16_rne(dz)
        dws[l] = oracle.gemm_bf16(hs[l], dz16, k, n, B, trans_a=True, trans_b=False, threads=8)
        if l > 0:
            dh = oracle.gemm_bf16(dz16, w16[l], B, k, n, trans_a=False, trans_b=True, threads=8)
    return loss, dws, dgs


def rel_fro(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("rows,d,V", [(64, 256, 1000), (48, 512, 2048), (16, 4096, 32000)])
def test_mlp_step_matches_oracle(rt, rows, d, V):
    """The last case has the layer widths and class count of the benchmark's MLP config on a reduced-row replica."""
    import torch
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    cfg = MlpConfig(d_in=d, hidden=[d, d, d], n_classes=V)
    tr = MlpTrainer(rt, cfg, rows)
    gx = torch.Generator(device="cuda"); gx.manual_seed(7)
    x = torch.randn((rows, d), generator=gx, device="cuda", dtype=torch.float32)
    gt = torch.Generator(device="cuda"); gt.manual_seed(8)
    targets = torch.randint(0, V, (rows,), generator=gt, device="cuda", dtype=torch.int32)
    for g in tr.gamma:      # non-trivial gammas exercise dgamma / dx properly
        g.copy_(1.0 + 0.1 * torch.randn(g.shape, device="cuda"))
    tr.forward_backward(x, targets)
    rt.synchronize()
    w16 = [w.view(torch.uint16).cpu().numpy() for w in tr.w16]
    gammas = [g.cpu().numpy() for g in tr.gamma]
    loss, dws, dgs = oracle_step(x.cpu().numpy(), targets.cpu().numpy().astype(np.uint32), w16, gammas, cfg.eps, 1.0 / rows)
    got_loss = tr.losses.cpu().numpy()
    assert np.abs(got_loss - loss).max() <= 1e-3 * np.abs(loss).max()
    assert abs(tr.mean_loss() - float(loss.mean())) <= 1e-3 * abs(float(loss.mean()))
    for i in range(4):
        assert rel_fro(tr.dw[i].cpu().numpy(), dws[i]) <= 5e-3, f"dW[{i}]"
    for i in range(3):
        got = tr.dgamma[i].cpu().numpy()
        assert np.abs(got - dgs[i]).max() <= 5e-3 * max(np.abs(dgs[i]).max(), 1e-6), f"dgamma[{i}]"
    # an optimizer step changes the master weights and refreshes the bf16 copies from them
    before = tr.master.clone()
    tr.optimizer_step()
    rt.synchronize()
    assert not torch.equal(before, tr.master)
    assert np.array_equal(tr.compute.view(torch.uint16).cpu().numpy(), oracle.f32_to_bf16_rne(tr.master.cpu().numpy()))


def test_mlp_loss_decreases(rt):
    """A few steps on a fixed batch reduce the loss (the reference's e2e check, src/ignis/tests.rs:395-477)."""
    import torch
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    cfg = MlpConfig(d_in=128, hidden=[128, 128, 128], n_classes=64, lr=3e-3)
    tr = MlpTrainer(rt, cfg, 256)
    x = torch.randn((256, 128), device="cuda")
    t = torch.randint(0, 64, (256,), device="cuda", dtype=torch.int32)
    losses = []
    for _ in range(12):
        tr.step(x, t)
        losses.append(tr.mean_loss())
    assert losses[-1] < losses[0] - 0.05, losses


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank, world, port, rows_total, q):
    import torch
    import torch.distributed as dist
    import t0_gpu_b200 as t
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    rt = t.GpuRuntime(rank)
    cfg = MlpConfig(d_in=256, hidden=[256, 256, 256], n_classes=512)
    rows = rows_total // world
    tr = MlpTrainer(rt, cfg, rows, rows_total=rows_total)
    g = torch.Generator(device="cuda"); g.manual_seed(7)
    x = torch.randn((rows_total, 256), generator=g, device="cuda")
    g2 = torch.Generator(device="cuda"); g2.manual_seed(8)
    tg = torch.randint(0, 512, (rows_total,), generator=g2, device="cuda", dtype=torch.int32)
    tr.forward_backward(x[rank * rows:(rank + 1) * rows].contiguous(), tg[rank * rows:(rank + 1) * rows].contiguous())
    rt.synchronize()
    loss = tr.mean_loss()
    if rank == 0:
        q.put((loss, tr.grads.cpu().numpy()))
    dist.barrier()
    dist.destroy_process_group()
    rt.close()


def test_data_parallel_two_ranks_match_one(rt):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    rows_total = 128
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, rows_total, q)) for r in range(2)]
    for p in procs:
        p.start()
    loss2, grads2 = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    cfg = MlpConfig(d_in=256, hidden=[256, 256, 256], n_classes=512)
    tr = MlpTrainer(rt, cfg, rows_total)
    g = torch.Generator(device="cuda"); g.manual_seed(7)
    x = torch.randn((rows_total, 256), generator=g, device="cuda")
    g2 = torch.Generator(device="cuda"); g2.manual_seed(8)
    tg = torch.randint(0, 512, (rows_total,), generator=g2, device="cuda", dtype=torch.int32)
    tr.forward_backward(x, tg)
    rt.synchronize()
    grads1 = tr.grads.cpu().numpy()
    assert abs(loss2 - tr.mean_loss()) <= 1e-5 * abs(loss2) + 1e-6
    assert rel_fro(grads2, grads1) <= 1e-3


def _sharded_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    import t0_gpu_b200 as t
    from t0_gpu_b200.mlp import MlpConfig, MlpTrainer

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    rt = t.GpuRuntime(rank)
    cfg = MlpConfig(d_in=256, hidden=[256, 256, 256], n_classes=512)
    rows_total = 128
    rows = rows_total // world
    g = torch.Generator(device="cuda"); g.manual_seed(7)
    x = torch.randn((rows_total, 256), generator=g, device="cuda")[rank * rows:(rank + 1) * rows].contiguous()
    g2 = torch.Generator(device="cuda"); g2.manual_seed(8)
    tg = torch.randint(0, 512, (rows_total,), generator=g2, device="cuda", dtype=torch.int32)[rank * rows:(rank + 1) * rows].contiguous()
    out = {}
    for mode in (False, True):
        tr = MlpTrainer(rt, cfg, rows, rows_total=rows_total, shard_optimizer=mode)
        assert tr.sharded == mode
        losses = []
        for _ in range(3):
            tr.step(x, tg)
            losses.append(tr.mean_loss())
        rt.synchronize()
        out[mode] = (losses, tr.gather_master().cpu().numpy(), tr.compute.view(torch.int16).cpu().numpy())
    if rank == 0:
        q.put(out)
    dist.barrier()
    dist.destroy_process_group()
    rt.close()


def test_sharded_optimizer_matches_replicated_optimizer():
    """Reduce-scatter + per-rank AdamW on a slice + all-gather gives the parameters of all-reduce + replicated AdamW:
    with two ranks every gradient sum has two terms, so the results are the same bits."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    (loss_r, master_r, bf16_r), (loss_s, master_s, bf16_s) = out[False], out[True]
    assert loss_r == loss_s and loss_r[2] < loss_r[0]
    assert np.array_equal(master_r, master_s)
    n_weights = 256 * 256 * 3 + 256 * 512        # the bf16 copies of the gammas (the tail) are not used by any kernel
    assert np.array_equal(bf16_r[:n_weights], bf16_s[:n_weights])
