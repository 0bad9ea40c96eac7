"""Column-sharded large GEMM over the GPUs of one node, one process per GPU.

B is split into contiguous N-column blocks, A is replicated, rank g computes C[:, block g].  The output
all-gather is folded into the GEMM epilogue: every rank holds a full row-major C[M, N] buffer that its peers
map through CUDA IPC, and the kernel stores each finished tile into its own buffer and straight into every
peer's buffer over NVLink (plain peer stores from the epilogue warps), so the transfer overlaps the math
tile by tile and no separate collective runs.  `torch.distributed` is used for the rendezvous only
(exchange of the 64-byte IPC handles, barriers).

There is no counterpart in the reference (single GPU; multi-GPU is a roadmap item there).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

from ._lib import lib
from .gemm_gen import GemmConfig
from .gpu_context import OUT_BF16, OUT_F32, GpuBuffer, GpuRuntime


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    col0: int       # first column of this rank's block
    n_local: int    # width of the block


def column_shard(n: int, world: int, rank: int, align: int = 64) -> ColumnShard:
    """Contiguous column blocks, widths multiples of `align` except possibly the last non-empty one.

    Blocks are as even as the alignment allows; with N a multiple of world*align every block is N/world.
    Trailing ranks may get an empty block when N is small."""
    if world < 1 or not (0 <= rank < world) or n < 0 or align < 1:
        raise ValueError(f"column_shard: bad arguments n={n} world={world} rank={rank} align={align}")
    units = (n + align - 1) // align            # aligned units, the last may be partial
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    col0 = min(u0 * align, n)
    col1 = min(u1 * align, n)
    return ColumnShard(rank, world, col0, col1 - col0)


def peer_order(rank: int, world: int) -> List[int]:
    """Order in which a rank's epilogue writes the destinations of a finished tile: its own buffer first (destination
    0 is the local store), then the peers starting at rank + 1, so that at any moment the ranks write to different
    peers and the traffic is spread over every GPU's NVLink ingress."""
    return [(rank + i) % world for i in range(world)]


def multi_dst_config(m: int, k: int, n_local: int, n_dst: int, num_sms: int = 148) -> GemmConfig:
    """The tile a sharded GEMM with `n_dst` destinations runs when no config is given (t0b_multi_dst_config)."""
    from .gemm_gen import GemmConfigC

    c = GemmConfigC()
    if lib().t0b_multi_dst_config(m, k, n_local, n_dst, num_sms, C.byref(c)) != 0:
        raise ValueError(f"multi_dst_config: bad arguments n_dst={n_dst}")
    return GemmConfig.from_c(c)


def exchange_handles(handle: bytes, group=None) -> List[bytes]:
    """All-gather one small byte string per rank over torch.distributed (any backend)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    out: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(out, handle, group=group)
    return [bytes(h) for h in out]


class _LibIpc:
    """CUDA IPC through the C ABI (t0b_ipc_export / open / close)."""

    def __init__(self, rt: GpuRuntime):
        self.rt = rt

    def export(self, ptr: int) -> bytes:
        h = (C.c_uint8 * 64)()
        self.rt._check(lib().t0b_ipc_export(self.rt.handle, ptr, h))
        return bytes(h)

    def open(self, handle: bytes) -> int:
        p = C.c_uint64()
        blob = (C.c_uint8 * 64).from_buffer_copy(handle)
        self.rt._check(lib().t0b_ipc_open(self.rt.handle, blob, C.byref(p)))
        return p.value

    def close(self, ptr: int) -> None:
        lib().t0b_ipc_close(self.rt.handle, ptr)


class ColumnShardedGemm:
    """C[M, N] = A[M, K] * B[K, N] with B column-sharded; each rank ends with the full C.

    a:        this rank's copy of A (bf16, [M, K] row-major)
    b_shard:  B[:, col0 : col0 + n_local] as its own row-major [K, n_local] buffer (bf16)
    c:        this rank's full output buffer [M, N] (bf16 or f32), from GpuRuntime.alloc

    Ordering contract.  `run()` launches THIS rank's kernel, which writes this rank's column block into every rank's
    C.  When it returns (even with async_=False) only this rank's own stores are known to be done: the other ranks'
    stores into this rank's C may still be in flight.  The full C is valid after `finish()`, which waits for this
    rank's kernel and then for every other rank to have done the same (a barrier of the group).  `close()` performs
    the same wait before any mapping is closed and before this rank's C can be released, so that no peer's
    epilogue is still storing into memory that goes away; every rank must call it (it is a collective).
    """

    def __init__(self, rt: GpuRuntime, m: int, n: int, k: int, out_dtype: int = OUT_BF16, group=None,
                 cfg: Optional[GemmConfig] = None, ipc=None):
        import torch.distributed as dist

        self.rt, self.m, self.n, self.k, self.out_dtype, self.group, self.cfg = rt, m, n, k, out_dtype, group, cfg
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.shard = column_shard(n, self.world, self.rank)
        self.ipc = ipc if ipc is not None else _LibIpc(rt)
        elem = 2 if out_dtype == OUT_BF16 else 4
        self.c = rt.alloc(m * n * elem)
        self._peer_ptrs: List[int] = []
        self._opened: List[int] = []
        self._closed = False
        self._map_peers()

    def _barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier(group=self.group)

    def _map_peers(self) -> None:
        if self.world == 1:
            self._peer_ptrs = [self.c.gpu_addr()]
            return
        handles = exchange_handles(self.ipc.export(self.c.gpu_addr()), self.group)
        ptrs = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                ptrs.append(self.c.gpu_addr())
                continue
            p = self.ipc.open(hb)
            ptrs.append(p)
            self._opened.append(p)
        self._peer_ptrs = [ptrs[r] for r in peer_order(self.rank, self.world)]

    def run(self, a: GpuBuffer, b_shard: GpuBuffer, async_: bool = True, gather: bool = True,
            rows: Optional[Sequence[int]] = None) -> None:
        """Launch this rank's GEMM.  With gather=False only the local C is written (GEMM-only timing).
        rows = (first_row, count) restricts the launch to a strip of rows of A and C (a caller that streams C to the
        host strip by strip).  The full C is NOT valid on return: call finish() before reading it."""
        if self._closed:
            raise RuntimeError("ColumnShardedGemm.run after close()")
        s = self.shard
        if s.n_local == 0:
            return
        r0, nrows = (0, self.m) if rows is None else (int(rows[0]), int(rows[1]))
        if r0 < 0 or nrows < 0 or r0 + nrows > self.m:
            raise ValueError(f"ColumnShardedGemm.run: rows {rows} outside 0..{self.m}")
        if nrows == 0:
            return
        elem = 2 if self.out_dtype == OUT_BF16 else 4
        dsts = self._peer_ptrs if gather else self._peer_ptrs[:1]
        arr = (C.c_uint64 * len(dsts))(*[p + r0 * self.n * elem for p in dsts])
        cp = C.byref(self.cfg.to_c()) if self.cfg is not None else None
        self.rt._check(lib().t0b_gemm_multi_dst(self.rt.handle, cp, 0, 0, a.gpu_addr() + r0 * self.k * 2, b_shard.gpu_addr(),
                                                arr, len(dsts), nrows, s.n_local, self.k, self.k, s.n_local, self.n,
                                                s.col0, self.out_dtype, int(async_)))

    def run_panels(self, a: GpuBuffer, b_shard: GpuBuffer, panels: int = 8) -> None:
        """The same product with the gather on the copy engines: the GEMM is launched panel by panel (row strips of
        A and C) with this rank's buffer as its only destination, and every finished panel is copied to each peer by
        t0b_copy_d2d_async on a side stream, peer (rank + 1) first, while the next panel is multiplied.  At any moment
        a rank sends to one peer, so the ranks' transfers form a permutation of the GPUs.  Same bits as run()."""
        if self._closed:
            raise RuntimeError("ColumnShardedGemm.run_panels after close()")
        s = self.shard
        if s.n_local == 0:
            return
        elem = 2 if self.out_dtype == OUT_BF16 else 4
        rows_per = (self.m + panels - 1) // panels
        rows_per = (rows_per + 255) // 256 * 256
        width = s.n_local * elem
        pitch = self.n * elem
        for r0 in range(0, self.m, rows_per):
            nrows = min(rows_per, self.m - r0)
            self.run(a, b_shard, async_=True, gather=False, rows=(r0, nrows))
            off = (r0 * self.n + s.col0) * elem
            for peer in self._peer_ptrs[1:]:
                self.rt._check(lib().t0b_copy_d2d_async(self.rt.handle, peer + off, pitch, self._peer_ptrs[0] + off, pitch,
                                                        width, nrows))

    def finish(self) -> None:
        """Collective: wait for this rank's kernel, then for every rank's.  After it every rank's C is complete."""
        self.rt.synchronize()
        self._barrier()

    def close(self) -> None:
        """Collective: finish(), then unmap the peers' buffers, then (after a second barrier, when every rank has
        unmapped) release this rank's C."""
        if self._closed:
            return
        self._closed = True
        self.finish()
        for p in self._opened:
            self.ipc.close(p)
        self._opened = []
        self._barrier()
        if self.c is not None:
            self.c.release()
            self.c = None
