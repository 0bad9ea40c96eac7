"""Host-side mirror of the reference runtime objects callers touch on the GEMM path:
`GpuRuntime` (src/ignis/gpu_context.rs:30-106, 113-483) and `GpuBuffer` (src/kfd/mod.rs:947-1061),
over the C ABI.  Errors surface as `T0Error` carrying the library's message (the reference returns
`Result<_, String>`); a CUDA error poisons the runtime like a queue timeout does in the reference."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from ._lib import lib
from .gemm_gen import GemmConfig


class T0Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[t0b {code}] {message}")
        self.code = code
        self.message = message


OUT_F32, OUT_BF16 = 0, 1


class GpuBuffer:
    """Device memory handle.  `write`/`read` are explicit copies (the reference maps VRAM into the host and
    tests read results through `host_ptr`); dropping the last reference frees the memory."""

    def __init__(self, rt: "GpuRuntime", addr: int, size: int, owned: bool = True):
        self._rt = rt
        self._addr = addr
        self._size = size
        self._owned = owned

    def gpu_addr(self) -> int:
        return self._addr

    def size(self) -> int:
        return self._size

    def write(self, data) -> None:
        buf = np.ascontiguousarray(data)
        if buf.nbytes > self._size:
            raise AssertionError(f"GpuBuffer.write: {buf.nbytes} bytes into a {self._size}-byte buffer")
        self._rt._check(lib().t0b_memcpy_h2d(self._rt._ctx, self._addr, buf.ctypes.data, buf.nbytes))

    def read(self, out: np.ndarray) -> np.ndarray:
        if out.nbytes > self._size:
            raise AssertionError(f"GpuBuffer.read: {out.nbytes} bytes from a {self._size}-byte buffer")
        assert out.flags["C_CONTIGUOUS"]
        self._rt._check(lib().t0b_memcpy_d2h(self._rt._ctx, out.ctypes.data, self._addr, out.nbytes))
        return out

    def read_as(self, dtype, count: int) -> np.ndarray:
        return self.read(np.empty(count, dtype=dtype))

    def zero(self) -> None:
        self._rt._check(lib().t0b_memset0(self._rt._ctx, self._addr, self._size))
        self._rt.synchronize()

    def release(self) -> None:
        if self._owned and self._addr and self._rt._ctx:
            lib().t0b_free(self._rt._ctx, self._addr)
        self._addr = 0

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class GpuRuntime:
    """One device + one in-order stream + a size-keyed buffer pool."""

    def __init__(self, device: int = 0):
        self._ctx = C.c_void_p()
        rc = lib().t0b_ctx_create(device, C.byref(self._ctx))
        if rc != 0:
            self._ctx = None
            raise T0Error(rc, "GPU init failed: no usable sm_100a CUDA device (there is no CPU fallback)")

    @staticmethod
    def new(device: int = 0) -> "GpuRuntime":
        return GpuRuntime(device)

    # ------------------------------------------------------------------ plumbing
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise T0Error(rc, lib().t0b_last_error(self._ctx).decode())

    @property
    def handle(self):
        return self._ctx

    def close(self) -> None:
        if self._ctx:
            lib().t0b_ctx_destroy(self._ctx)
            self._ctx = None

    def set_stream(self, cuda_stream: int) -> None:
        self._check(lib().t0b_ctx_set_stream(self._ctx, C.c_void_p(cuda_stream)))

    def num_sms(self) -> int:
        return lib().t0b_num_sms(self._ctx)

    def set_sm_limit(self, sms: int) -> None:
        """GEMM kernels occupy at most `sms` SMs (0 = all), leaving the rest to kernels running beside them."""
        self._check(lib().t0b_set_sm_limit(self._ctx, sms))

    def is_poisoned(self) -> bool:
        return bool(lib().t0b_is_poisoned(self._ctx))

    def device_status(self, clear: bool = False) -> int:
        return lib().t0b_device_status(self._ctx, int(clear))

    def launch_count(self) -> int:
        return lib().t0b_launch_count(self._ctx)

    # ------------------------------------------------------------------ memory (gpu_context.rs:437-483)
    def alloc(self, size: int) -> GpuBuffer:
        p = C.c_uint64()
        self._check(lib().t0b_alloc(self._ctx, size, C.byref(p)))
        return GpuBuffer(self, p.value, size)

    def alloc_zero(self, size: int) -> GpuBuffer:
        p = C.c_uint64()
        self._check(lib().t0b_alloc_zero(self._ctx, size, C.byref(p)))
        return GpuBuffer(self, p.value, size)

    def alloc_f32(self, n: int) -> GpuBuffer:
        """n floats, at least 512 bytes, zero-filled (gpu_context.rs:449-454)."""
        return self.alloc_zero(max(n * 4, 512))

    def recycle(self, buf: GpuBuffer) -> None:
        self._check(lib().t0b_recycle(self._ctx, buf._addr))
        buf._addr = 0

    def upload(self, data) -> GpuBuffer:
        arr = np.ascontiguousarray(data)
        b = self.alloc(max(arr.nbytes, 16))
        b.write(arr)
        return b

    def upload_f32(self, data) -> GpuBuffer:
        return self.upload(np.ascontiguousarray(data, dtype=np.float32))

    def write_f32(self, buf: GpuBuffer, data) -> None:
        buf.write(np.ascontiguousarray(data, dtype=np.float32))

    def read_f32(self, buf: GpuBuffer, n: int) -> np.ndarray:
        return buf.read_as(np.float32, n)

    def pool_stats(self) -> dict:
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        lib().t0b_pool_stats(self._ctx, C.byref(a), C.byref(b), C.byref(c))
        return {"cached_bytes": a.value, "hits": b.value, "misses": c.value}

    # ------------------------------------------------------------------ bf16 weight cache (gpu_context.rs:392-432)
    def get_or_create_bf16(self, tensor_id: int, f32_buf: GpuBuffer, n_elems: int) -> GpuBuffer:
        """`GpuRuntime::get_or_create_bf16(tensor_id, f32_buf, n_elems, convert_kernel)`: the cached bf16 copy of an f32
        weight buffer, converted on the device on first use (no convert-kernel argument: the library owns the kernel).
        The returned handle is borrowed -- the cache owns the memory."""
        p = C.c_uint64()
        self._check(lib().t0b_get_or_create_bf16(self._ctx, tensor_id, f32_buf.gpu_addr(), n_elems, C.byref(p)))
        return GpuBuffer(self, p.value, n_elems * 2, owned=False)

    def invalidate_bf16(self, tensor_id: int) -> None:
        """Call after a weight update (gpu_context.rs:420-424)."""
        self._check(lib().t0b_invalidate_bf16(self._ctx, tensor_id))

    def clear_bf16_cache(self) -> None:
        self._check(lib().t0b_clear_bf16_cache(self._ctx))

    def bf16_cache_stats(self) -> dict:
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        lib().t0b_bf16_cache_stats(self._ctx, C.byref(a), C.byref(b), C.byref(c))
        return {"entries": a.value, "conversions": b.value, "hits": c.value}

    # ------------------------------------------------------------------ sync (gpu_context.rs:297-332)
    def synchronize(self) -> None:
        self._check(lib().t0b_sync(self._ctx))

    wait_idle = synchronize

    # ------------------------------------------------------------------ GEMM
    def gemm(self, a: GpuBuffer, b: GpuBuffer, c: GpuBuffer, m: int, n: int, k: int, *, cfg: Optional[GemmConfig] = None,
             trans_a: bool = False, trans_b: bool = True, lda: Optional[int] = None, ldb: Optional[int] = None,
             ldc: Optional[int] = None, out_dtype: int = OUT_F32, epilogue: int = 0, bias: Optional[GpuBuffer] = None,
             alpha: float = 1.0, workspace: Optional[GpuBuffer] = None, async_: bool = False) -> None:
        lda = lda if lda is not None else (m if trans_a else k)
        ldb = ldb if ldb is not None else (k if trans_b else n)
        ldc = ldc if ldc is not None else n
        cp = C.byref(cfg.to_c()) if cfg is not None else None
        self._check(lib().t0b_gemm(self._ctx, cp, int(trans_a), int(trans_b), _addr(a), _addr(b), _addr(c), m, n, k,
                                   lda, ldb, ldc, out_dtype, epilogue, _addr(bias), alpha, _addr(workspace),
                                   workspace.size() if workspace is not None else 0, int(async_)))

    def gemm_slabs(self, x: GpuBuffer, wt: GpuBuffer, y: GpuBuffer, m: int, n: int, k: int, split_k: int,
                   cfg: Optional[GemmConfig] = None, async_: bool = False) -> None:
        cp = C.byref(cfg.to_c()) if cfg is not None else None
        self._check(lib().t0b_gemm_slabs(self._ctx, cp, _addr(x), _addr(wt), _addr(y), m, n, k, split_k, int(async_)))

    def splitk_reduce(self, partial: GpuBuffer, split_k: int, m: int, n: int, c: GpuBuffer, out_dtype: int = OUT_F32,
                      epilogue: int = 0, bias: Optional[GpuBuffer] = None, async_: bool = False) -> None:
        self._check(lib().t0b_splitk_reduce(self._ctx, _addr(partial), split_k, m, n, m * n, n, _addr(c), n, out_dtype,
                                            epilogue, _addr(bias), 1.0, int(async_)))

    def ensure_kernel_t0(self, name: str, build, workgroup_size=None, lds_size: int = 0):
        """`GpuRuntime::ensure_kernel_t0(name, || build(), wg, lds)` (gpu_context.rs:196-262): build once per name and
        keep the kernel for the life of the runtime.  `build` returns a `T0Kernel` (gemm_gen::generate) or a
        `TileKernel` (tile_ir::lower_gemm); workgroup size and LDS size are accepted and not needed here."""
        cache = self.__dict__.setdefault("_kernels", {})
        if name not in cache:
            cache[name] = build()
        return cache[name]

    def dispatch(self, kernel, grid, kernargs: bytes) -> None:
        """`GpuRuntime::dispatch(kernel, grid, kernargs)`: synchronous (gpu_context.rs:264-288).  `kernel` is a
        GemmConfig / T0Kernel / GpuKernel (40/44/48-byte gemm_gen blobs) or a tile_ir TileKernel / TileGemm."""
        self._dispatch(kernel, grid, kernargs, False)

    def dispatch_async(self, kernel, grid, kernargs: bytes) -> None:
        self._dispatch(kernel, grid, kernargs, True)

    def dispatch_bench(self, kernel, grid, kernargs: bytes) -> float:
        """`GpuRuntime::dispatch_bench` (gpu_context.rs:297-307): the reference's low-overhead submit + spin-wait for
        benchmarks.  Here: one launch bracketed by CUDA events on the stream; returns the device time in milliseconds
        (the reference returns nothing and leaves the timing to the caller's wall clock)."""
        import torch

        stream = torch.cuda.ExternalStream(lib().t0b_ctx_stream(self._ctx) or 0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        self._dispatch(kernel, grid, kernargs, True)
        e1.record(stream)
        self.synchronize()
        return e0.elapsed_time(e1)

    def _dispatch(self, kernel, grid, kernargs, async_):
        blob = (C.c_uint8 * len(kernargs)).from_buffer_copy(kernargs)
        spec = getattr(kernel, "spec", None)
        if spec is None and hasattr(kernel, "acc_swap"):
            spec = kernel
        if spec is not None:
            g = (C.c_uint32 * 3)(grid[0], grid[1], grid[2] if len(grid) > 2 else 1)
            self._check(lib().t0b_tile_dispatch(self._ctx, C.byref(spec.to_c()), g, blob, len(kernargs), int(async_)))
            return
        cfg = getattr(kernel, "cfg", kernel)
        self._check(lib().t0b_dispatch_kernargs(self._ctx, C.byref(cfg.to_c()), grid[0], grid[1], blob, len(kernargs),
                                                int(async_)))

    def gemm_time(self, a: GpuBuffer, b: GpuBuffer, c: GpuBuffer, m: int, n: int, k: int, *, cfg=None, trans_a=False,
                  trans_b=True, out_dtype=OUT_F32, warmup=3, iters=10) -> float:
        lda = m if trans_a else k
        ldb = k if trans_b else n
        ms = C.c_float()
        cp = C.byref(cfg.to_c()) if cfg is not None else None
        self._check(lib().t0b_gemm_time(self._ctx, cp, int(trans_a), int(trans_b), _addr(a), _addr(b), _addr(c), m, n, k,
                                        lda, ldb, n, out_dtype, warmup, iters, C.byref(ms)))
        return ms.value

    def tune(self, m: int, n: int, k: int, trans_a=False, trans_b=True, out_dtype=OUT_F32):
        """GemmTuner::tune(rt, m, n, k) (src/t0/auto_gemm.rs:82): returns (best config, TFLOP/s)."""
        from ._lib import GemmConfigC
        out = GemmConfigC()
        tf = C.c_float()
        self._check(lib().t0b_tune(self._ctx, m, n, k, int(trans_a), int(trans_b), out_dtype, C.byref(out), C.byref(tf)))
        return GemmConfig.from_c(out), tf.value

    def selftest_bounded_wait(self, limit_ns: int) -> int:
        return lib().t0b_selftest_bounded_wait(self._ctx, limit_ns)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------ the low-level handshake the examples drive
# generate(&cfg).compile(Target) -> blob; GpuKernel::load(&device, &blob, &KernelLoadConfig);
# queue.submit(&kernel, [gx, gy, 1], kernargs); queue.wait_idle()   (examples/test_gemm_correctness.rs:93-188)

class Target:
    SM100A = "sm_100a"
    GFX1100 = "sm_100a"      # accepted alias: code written against the reference keeps compiling


class T0Kernel:
    """What `gemm_gen::generate(&cfg)` returns here: a handle naming a precompiled sm_100a kernel variant."""

    def __init__(self, cfg: GemmConfig):
        self.cfg = cfg

    def compile(self, target=Target.SM100A) -> bytes:
        """Nothing is compiled at run time; the "ELF" is an opaque descriptor of the config."""
        import json
        from dataclasses import asdict
        d = asdict(self.cfg)
        d["transpose"], d["epilogue"] = int(self.cfg.transpose), int(self.cfg.epilogue)
        return b"T0B200\0" + json.dumps(d, sort_keys=True).encode()


def generate(cfg: GemmConfig) -> T0Kernel:
    if not cfg.is_feasible():
        raise ValueError(f"[gemm_gen] config {cfg.name()} cannot be mapped onto the sm_100a kernel family")
    return T0Kernel(cfg)


class KernelLoadConfig:
    def __init__(self, workgroup_size=(192, 1, 1), lds_size: int = 0):
        self.workgroup_size, self.lds_size = workgroup_size, lds_size    # accepted, not needed on B200


class GpuKernel:
    def __init__(self, cfg: GemmConfig):
        self.cfg = cfg

    @staticmethod
    def load(rt, blob: bytes, load_cfg: Optional[KernelLoadConfig] = None) -> "GpuKernel":
        """`GpuKernel::load(&device, &elf, &KernelLoadConfig{..})`; `rt` is a GpuRuntime or a KfdDevice."""
        import json
        from .gemm_gen import EpilogueOp, GemmTranspose
        if not blob.startswith(b"T0B200\0"):
            raise T0Error(-1, "GpuKernel.load: not a t0b200 kernel descriptor")
        d = json.loads(blob[7:].decode())
        d["transpose"], d["epilogue"] = GemmTranspose(d["transpose"]), EpilogueOp(d["epilogue"])
        return GpuKernel(GemmConfig(**d))


class KernargBuffer:
    """One kernarg slot of a `DispatchPool`.  In the reference this is a 256-byte uncached GPU buffer the command
    processor reads; a CUDA launch takes its arguments by value, so the slot is host memory with the same
    `write` / `read` / `size` surface, and `AqlQueue.submit` reads the blob out of it at submission."""

    SLOT_BYTES = 256

    def __init__(self):
        self._data = bytearray(self.SLOT_BYTES)
        self._len = 0

    def write(self, data: bytes) -> None:
        if len(data) > self.SLOT_BYTES:
            raise AssertionError(f"KernargBuffer.write: {len(data)} bytes into a {self.SLOT_BYTES}-byte slot")
        self._data[:len(data)] = data
        self._len = len(data)

    def read(self) -> bytes:
        return bytes(self._data[:self._len])

    def size(self) -> int:
        return self.SLOT_BYTES


class DispatchPool:
    """`kfd::DispatchPool` (src/kfd/mod.rs:2853-2930): an auto-growing ring of kernarg slots addressed by index.
    `new(device, initial_slots)` pre-creates `initial_slots` slots (0 = 1024); any index may be used, missing slots
    are created on access.  The completion signal of the reference has no counterpart: completion is the stream's."""

    def __init__(self, device, initial_slots: int = 0):
        self.device = device
        n = 1024 if initial_slots == 0 else initial_slots
        self._ring = [KernargBuffer() for _ in range(n)]

    @staticmethod
    def new(device, initial_slots: int = 0) -> "DispatchPool":
        return DispatchPool(device, initial_slots)

    def _ensure_slot(self, idx: int) -> None:
        if idx < 0:
            raise IndexError("DispatchPool: negative slot index")
        while idx >= len(self._ring):
            self._ring.append(KernargBuffer())

    def get_kernargs(self, idx: int) -> KernargBuffer:
        self._ensure_slot(idx)
        return self._ring[idx]

    def write_kernargs(self, idx: int, data: bytes) -> KernargBuffer:
        """Write the blob into slot `idx` (created on demand) and return the slot (mod.rs:2901-2910)."""
        buf = self.get_kernargs(idx)
        buf.write(data)
        return buf

    def dispatch(self, queue: "AqlQueue", kernel, grid, ka_idx: int) -> None:
        """Submit with the blob of slot `ka_idx` and wait for completion (mod.rs:2912-2925)."""
        queue.submit(kernel, grid, self.get_kernargs(ka_idx))
        queue.wait_idle()

    def len(self) -> int:
        return len(self._ring)

    __len__ = len

    def capacity(self) -> int:
        return len(self._ring)


class AqlQueue:
    """`queue.submit` + `queue.wait_idle` over the runtime's stream.  `kernargs` is a blob or a `DispatchPool` slot."""

    def __init__(self, rt: "GpuRuntime"):
        self.rt = rt

    def submit(self, kernel: GpuKernel, grid, kernargs) -> None:
        blob = kernargs.read() if isinstance(kernargs, KernargBuffer) else kernargs
        self.rt.dispatch_async(kernel.cfg, (grid[0], grid[1]), blob)

    def wait_idle(self) -> None:
        self.rt.synchronize()


class KfdDevice:
    """The device handle the reference's examples open first (`KfdDevice::open()`, src/kfd/mod.rs): here a thin view
    of a `GpuRuntime` with the three calls those examples make -- `create_queue`, `alloc_vram`, and being passed to
    `GpuKernel::load` / `DispatchPool::new`."""

    def __init__(self, rt: "GpuRuntime"):
        self.rt = rt

    @staticmethod
    def open(device: int = 0, rt: Optional["GpuRuntime"] = None) -> "KfdDevice":
        return KfdDevice(rt if rt is not None else GpuRuntime(device))

    def create_queue(self) -> AqlQueue:
        return AqlQueue(self.rt)

    def alloc_vram(self, size: int) -> GpuBuffer:
        return self.rt.alloc(size)


def _addr(b) -> int:
    if b is None:
        return 0
    if isinstance(b, int):
        return b
    return b.gpu_addr()
