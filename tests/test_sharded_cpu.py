"""Host-side logic of the column-sharded GEMM, on CPU: the shard arithmetic and the handle exchange between
two `gloo` ranks (the GPU kernels are not involved)."""
import os
import socket

import pytest

from t0_gpu_b200.sharded import column_shard, exchange_handles


def test_column_shards_tile_the_columns():
    for n in (32768, 8192, 4096, 1000, 130, 64, 7, 0):
        for world in (1, 2, 4, 8):
            shards = [column_shard(n, world, r) for r in range(world)]
            assert shards[0].col0 == 0
            assert sum(s.n_local for s in shards) == n
            for a, b in zip(shards, shards[1:]):
                assert a.col0 + a.n_local == b.col0                      # contiguous, in rank order
            for s in shards:
                assert s.col0 % 64 == 0 or s.n_local == 0                 # TMA-friendly block starts
            if n % (64 * world) == 0:
                assert all(s.n_local == n // world for s in shards)       # the benchmark case: equal blocks
    s = column_shard(32768, 8, 3)
    assert (s.col0, s.n_local) == (3 * 4096, 4096)
    with pytest.raises(ValueError):
        column_shard(128, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        mine = bytes([rank]) * 64                                         # stands in for a 64-byte IPC handle
        got = exchange_handles(mine)
        shard = column_shard(1024, world, rank)
        # destination order used by the fused epilogue: own buffer first, then the peers in rank order
        order = [rank] + [r for r in range(world) if r != rank]
        q.put((rank, [h[0] for h in got], len(got[0]), shard.col0, shard.n_local, order))
    finally:
        dist.destroy_process_group()


def test_handle_exchange_between_two_gloo_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    world = 2
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, firsts, hlen, col0, n_local, order in results:
        assert firsts == [0, 1] and hlen == 64                            # every rank sees every handle, in rank order
        assert (col0, n_local) == (rank * 512, 512)
        assert order[0] == rank and sorted(order) == [0, 1]
