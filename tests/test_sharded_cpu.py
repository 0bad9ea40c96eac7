"""Host-side logic of the multi-GPU paths, on CPU: the column-shard arithmetic and the handle exchange of the sharded
GEMM between two `gloo` ranks, the peer write order, and the unit / slice arithmetic of the data-parallel MLP step with
its sharded optimizer (emulated with gloo collectives and the oracle's AdamW; the GPU kernels are not involved)."""
import os
import socket

import pytest

from t0_gpu_b200.sharded import column_shard, exchange_handles, peer_order


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


def test_multi_destination_gemm_uses_the_double_buffered_tile():
    """With peers the epilogue issues NVLink stores, so once the link time matters the sharded benchmark shape must not
    run on a tile whose epilogue is exposed (256x512 / 512x256 keep both TMEM accumulators for one tile)."""
    from t0_gpu_b200.sharded import multi_dst_config

    m, k = 32768, 8192
    for world in (2, 4, 8):
        n_local = 32768 // world
        two_acc = {(256, 512), (512, 256)}      # the tiles that keep both TMEM accumulators for one tile
        alone = multi_dst_config(m, k, n_local, 1)
        assert (alone.tile_m, alone.tile_n) in two_acc and not alone.split_k           # what one GPU runs (shipped table)
        fused = multi_dst_config(m, k, n_local, world)
        if world == 2:       # link time / math time = 0.25: the faster math tile wins (measured)
            assert (fused.tile_m, fused.tile_n) in two_acc and not fused.split_k
        else:                # 0.75 and 1.8: the stores must overlap the next main loop
            assert (fused.tile_m, fused.tile_n, fused.wg_size) == (256, 256, 192) and not fused.split_k
    small = multi_dst_config(256, 256, 256, 2)                                    # small tiles are left alone
    assert small.tile_m <= 256 and small.tile_n <= 256 and not small.split_k
    with pytest.raises(ValueError):
        multi_dst_config(m, k, 4096, 9)


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
        order = peer_order(rank, world)      # destination order used by the fused epilogue
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


class _FakeBuf:
    def __init__(self, log, addr):
        self.log, self.addr = log, addr

    def gpu_addr(self):
        return self.addr

    def release(self):
        self.log.append("free_c")


class _FakeRt:
    """Stands in for GpuRuntime: records the order of the calls the sharded GEMM makes."""

    def __init__(self, log, rank):
        self.log, self.rank, self.handle = log, rank, None

    def alloc(self, size):
        self.log.append("alloc_c")
        return _FakeBuf(self.log, 0x1000 * (self.rank + 1))

    def synchronize(self):
        self.log.append("sync")


class _FakeIpc:
    def __init__(self, log, rank):
        self.log, self.rank = log, rank

    def export(self, ptr):
        self.log.append("export")
        return bytes([self.rank]) * 64

    def open(self, handle):
        self.log.append(f"open{handle[0]}")
        return 0x100000 * (handle[0] + 1)

    def close(self, ptr):
        self.log.append(f"close{ptr // 0x100000 - 1}")


def _order_worker(rank: int, world: int, port: int, q):
    import torch.distributed as dist

    import t0_gpu_b200.sharded as sh

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        log = []
        real_barrier = dist.barrier

        def logged_barrier(*a, **k):
            log.append("barrier")
            return real_barrier(*a, **k)

        dist.barrier = logged_barrier
        op = sh.ColumnShardedGemm(_FakeRt(log, rank), 256, 1024, 64, ipc=_FakeIpc(log, rank))
        ptrs = list(op._peer_ptrs)
        op.finish()
        op.close()
        op.close()                      # idempotent
        closed_run = False
        try:
            op.run(None, None)
        except RuntimeError:
            closed_run = True
        q.put((rank, log, ptrs, closed_run))
    finally:
        dist.destroy_process_group()


def test_sharded_gemm_orders_peer_stores_before_unmapping_and_freeing():
    """finish() = wait for the local kernel, then a barrier; close() = the same, then the unmaps, then another barrier,
    and only then this rank's C goes away -- no peer can still be storing into it."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_order_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, log, ptrs, closed_run in results:
        other = 1 - rank
        assert log == ["alloc_c", "export", f"open{other}",            # construction: map the peer's C
                       "sync", "barrier",                               # finish()
                       "sync", "barrier", f"close{other}", "barrier", "free_c"]   # close()
        assert ptrs == [0x1000 * (rank + 1), 0x100000 * (other + 1)]    # own buffer first, then the peer's mapping
        assert closed_run


def test_peer_order_spreads_the_writes():
    for world in (1, 2, 4, 8):
        orders = [peer_order(r, world) for r in range(world)]
        for r, o in enumerate(orders):
            assert o[0] == r and sorted(o) == list(range(world))          # own buffer first, every rank once
        for step in range(world):                                         # at every step the ranks hit distinct targets
            assert sorted(o[step] for o in orders) == list(range(world))


def test_exchange_units_cover_the_parameters():
    from t0_gpu_b200.mlp import exchange_units, shard_range

    dims = [(4096, 4096), (4096, 4096), (4096, 4096), (4096, 32000)]
    hidden = [4096, 4096, 4096]
    n_params = sum(k * n for k, n in dims) + sum(hidden)
    for want_shard in (False, True):
        units, layer_units, gamma_unit = exchange_units(dims, hidden, want_shard)
        assert units[0][0] == 0 and units[-1][0] + units[-1][1] == n_params
        for (o0, n0), (o1, _) in zip(units, units[1:]):
            assert o0 + n0 == o1                                          # contiguous, no gaps, no overlap
        assert [len(x) for x in layer_units] == ([1, 1, 1, 4] if want_shard else [1, 1, 1, 1])
        assert gamma_unit == len(units) - 1 and units[gamma_unit][1] == sum(hidden)
        assert sum(units[u][1] for u in layer_units[3]) == 4096 * 32000
        for world in (2, 4, 8):
            for unit in units:
                assert unit[1] % world == 0
                slices = [shard_range(unit, r, world) for r in range(world)]
                assert slices[0][0] == unit[0] and slices[-1][1] == unit[0] + unit[1]
                for a, b in zip(slices, slices[1:]):
                    assert a[1] == b[0]
    # a layer whose row count is not a multiple of the panel count stays in one piece
    units, layer_units, _ = exchange_units([(6, 10), (7, 9)], [10], True)
    assert layer_units == [[0], [1]] and units[1] == (60, 63)


def _dp_worker(rank: int, world: int, port: int, q):
    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle
    from t0_gpu_b200.mlp import exchange_units, shard_range

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        dims, hidden = [(8, 12), (12, 12), (12, 16)], [12, 12]
        units, _, _ = exchange_units(dims, hidden, True)
        n = units[-1][0] + units[-1][1]
        rng = np.random.default_rng(3)                                   # same parameters on every rank
        params = rng.standard_normal(n).astype(np.float32)
        local_grads = np.random.default_rng(100 + rank).standard_normal(n).astype(np.float32)
        hp = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, t=1)
        # replicated optimizer: all-reduce, then AdamW over everything
        g = torch.from_numpy(local_grads.copy())
        dist.all_reduce(g)
        full_p, _, _ = oracle.adamw_step(params, g.numpy(), np.zeros(n, np.float32), np.zeros(n, np.float32), **hp)
        # sharded optimizer: every rank updates its slice of every unit (the reduce-scatter is emulated by slicing the
        # all-reduced gradient, which is what it delivers), then the slices are gathered
        out = torch.from_numpy(params.copy())
        for unit in units:
            lo, hi = shard_range(unit, rank, world)
            p, _, _ = oracle.adamw_step(params[lo:hi], g.numpy()[lo:hi], np.zeros(hi - lo, np.float32), np.zeros(hi - lo, np.float32), **hp)
            pieces = [torch.empty(hi - lo) for _ in range(world)]
            dist.all_gather(pieces, torch.from_numpy(p))
            out[unit[0]:unit[0] + unit[1]] = torch.cat(pieces)
        q.put((rank, bool(np.array_equal(out.numpy(), full_p)), float(np.abs(full_p - params).max())))
    finally:
        dist.destroy_process_group()


def test_sharded_optimizer_indexing_between_two_gloo_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, same, moved in results:
        assert same and moved > 0          # gathered slices == the replicated update, and the update did something
