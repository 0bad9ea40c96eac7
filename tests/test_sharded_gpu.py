"""The column-sharded GEMM with the all-gather fused into the epilogue, on two GPUs (skipped with fewer): every rank
ends with the same full C, equal to the single-GPU result bit for bit."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, q):
    import torch
    import torch.distributed as dist
    import t0_gpu_b200 as t
    from t0_gpu_b200._lib import lib
    from t0_gpu_b200.sharded import ColumnShardedGemm

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    rt = t.GpuRuntime(rank)
    g = torch.Generator(device=dev); g.manual_seed(4321)
    a = (torch.randn((m, k), generator=g, device=dev) / k ** 0.5).to(torch.bfloat16)
    g.manual_seed(4322)
    b = (torch.randn((k, n), generator=g, device=dev) / k ** 0.5).to(torch.bfloat16)
    op = ColumnShardedGemm(rt, m, n, k, out_dtype=t.OUT_BF16)
    sh = op.shard
    b_sh = b[:, sh.col0:sh.col0 + sh.n_local].contiguous()

    class Buf:
        def __init__(self, tensor):
            self.t = tensor

        def gpu_addr(self):
            return self.t.data_ptr()

    dist.barrier()
    op.run(Buf(a), Buf(b_sh), async_=False, gather=True)
    dist.barrier()                 # every rank's peer stores have been issued and completed
    rt.synchronize()
    full = np.empty(m * n, np.uint16)
    op.c.read(full)
    if rank == 0:
        # single-GPU result of the whole product on this rank
        c1 = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        rt._check(lib().t0b_gemm(rt.handle, None, 0, 0, a.data_ptr(), b.data_ptr(), c1.data_ptr(), m, n, k, k, n, n, 1, 0, 0,
                                 1.0, 0, 0, 0))
        q.put(("single", c1.view(torch.uint16).cpu().numpy().ravel()))
    q.put((rank, full))
    dist.barrier()
    op.close()
    dist.destroy_process_group()
    rt.close()


@pytest.mark.parametrize("m,n,k", [(1024, 2048, 512), (600, 1000, 264)])
def test_two_rank_sharded_gemm_equals_single_gpu(m, n, k):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, m, n, k, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(3))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert np.array_equal(got[0], got[1])            # both ranks hold the same full C
    assert np.array_equal(got[0], got["single"])     # and it equals the one-GPU product, bit for bit
