// Runtime of libt0b200.so: context, stream, buffer pool, copies, status word, CUDA graphs.
// Stands where the reference has GpuRuntime + BufferPool (src/ignis/gpu_context.rs:30-106, 113-483) on top of
// the KFD queue/VRAM layer (src/kfd/mod.rs): a CUDA stream replaces the AQL queue and doorbell, cudaMalloc
// the VRAM mmap, a mapped status word the queue-timeout detection.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "t0b_internal.hpp"

namespace t0b {

int32_t set_error(t0b_ctx* ctx, int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) {
        std::lock_guard<std::recursive_mutex> lk(ctx->mu);
        ctx->last_error = buf;
        if (code == T0B_ERR_CUDA) ctx->poisoned = true;
    }
    return code;
}

int32_t check_cuda(t0b_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaSuccess) return T0B_OK;
    // The runtime also remembers the error per host thread; clear that copy so it cannot surface later as the
    // "last error" of an unrelated launch from another context.
    cudaGetLastError();
    return set_error(ctx, T0B_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

int32_t precheck(t0b_ctx* ctx) {
    if (!ctx) return T0B_ERR_INVALID;
    if (ctx->poisoned) {
        // Keep the message of the error that poisoned the context.
        return T0B_ERR_POISONED;
    }
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return check_cuda(ctx, e, "cudaSetDevice");
    return T0B_OK;
}

int take_device_status(t0b_ctx* ctx) {
    if (!ctx || !ctx->status_host) return 0;
    volatile int* w = reinterpret_cast<volatile int*>(ctx->status_host);
    const int st = *w;
    if (st != 0) {
        ctx->last_status = st;
        *w = 0;
    }
    return st;
}

int32_t finish(t0b_ctx* ctx, int32_t async, const char* what, int count) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
    ctx->launches += static_cast<uint64_t>(count);
    if (async || ctx->capturing) return T0B_OK;
    e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return check_cuda(ctx, e, what);
    const int st = take_device_status(ctx);
    if (st != 0) return set_error(ctx, T0B_ERR_DEVICE, "%s: device status %d (101-105: a bounded in-kernel wait ran out; 110: an index outside its table)", what, st);
    return T0B_OK;
}

}  // namespace t0b

using namespace t0b;

static size_t round4k(size_t b) { return (b + 4095) & ~static_cast<size_t>(4095); }

// A cached bf16 copy keyed by this device address (the default key of an f32 weight buffer) describes contents that are
// about to change or go away: drop it.  Copies under caller-chosen ids are the caller's to invalidate.
static void drop_bf16_of(t0b_ctx* ctx, uint64_t f32_addr) {
    if (ctx->bf16_cache.empty()) return;
    auto it = ctx->bf16_cache.find(f32_addr);
    if (it == ctx->bf16_cache.end()) return;
    const uint64_t copy = it->second.ptr;
    ctx->bf16_cache.erase(it);
    t0b_recycle(ctx, copy);
}

extern "C" {

int32_t t0b_ctx_create(int32_t device, t0b_ctx** out) {
    if (!out) return T0B_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0 || device < 0 || device >= count) {
        cudaGetLastError();
        return T0B_ERR_CUDA;   // no CPU fallback: without a usable CUDA device there is no context
    }
    t0b_ctx* ctx = new t0b_ctx();
    ctx->device = device;
    int32_t rc = check_cuda(ctx, cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop{};
    if (rc == T0B_OK) rc = check_cuda(ctx, cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (rc == T0B_OK && prop.major != 10) {
        rc = set_error(ctx, T0B_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                       prop.major, prop.minor);
    }
    if (rc == T0B_OK) {
        ctx->num_sms = prop.multiProcessorCount;
        if (const char* e = std::getenv("T0B_PDL")) ctx->pdl = std::atoi(e) != 0;
        if (const char* e = std::getenv("T0B_CLUSTER_SPLITK")) ctx->cluster_splitk = std::atoi(e) != 0;
        if (const char* e = std::getenv("T0B_WAIT_HINT_NS")) ctx->wait_hint_ns = static_cast<unsigned>(std::max(0, std::atoi(e)));
        if (const char* e = std::getenv("T0_FORCE_CONFIG")) ctx->force_config = e;
        if (const char* e = std::getenv("T0_DUMP_CONFIG")) ctx->dump_config = std::atoi(e) != 0;
        if (const char* e = std::getenv("T0B_RASTER_GROUP")) ctx->raster_group = std::max(0, std::atoi(e));
        rc = check_cuda(ctx, cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        ctx->stream = ctx->own_stream;
    }
    if (rc == T0B_OK) {
        rc = check_cuda(ctx, cudaHostAlloc(reinterpret_cast<void**>(&ctx->status_host), 64, cudaHostAllocMapped),
                        "cudaHostAlloc(status)");
        if (rc == T0B_OK) {
            std::memset(ctx->status_host, 0, 64);
            rc = check_cuda(ctx, cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->status_dev), ctx->status_host, 0),
                            "cudaHostGetDevicePointer");
        }
    }
    if (rc != T0B_OK) {
        t0b_ctx_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return T0B_OK;
}

void t0b_ctx_destroy(t0b_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->own_stream) cudaStreamSynchronize(ctx->own_stream);
    for (auto& g : ctx->graphs) cudaGraphExecDestroy(g.second);
    for (auto& kv : ctx->pool_free) cudaFree(kv.second);
    for (auto& kv : ctx->live) cudaFree(kv.first);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->h2d_stream) cudaStreamDestroy(ctx->h2d_stream);
    if (ctx->d2h_stream) cudaStreamDestroy(ctx->d2h_stream);
    if (ctx->p2p_stream) cudaStreamDestroy(ctx->p2p_stream);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
}

int32_t t0b_ctx_set_stream(t0b_ctx* ctx, void* s) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    cudaStream_t next = s ? static_cast<cudaStream_t>(s) : ctx->own_stream;
    if (next != ctx->stream && !ctx->capturing) {
        // Work queued on the old stream may still use buffers that were recycled to the pool (or the split-K
        // workspace); everything launched on the new stream is ordered behind it.
        cudaSetDevice(ctx->device);
        cudaEvent_t ev = nullptr;
        cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventRecord(ev, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(next, ev, 0);
        if (ev) cudaEventDestroy(ev);
        if (e != cudaSuccess) return check_cuda(ctx, e, "t0b_ctx_set_stream (ordering the new stream behind the old)");
    }
    ctx->stream = next;
    return T0B_OK;
}

void* t0b_ctx_stream(t0b_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }

const char* t0b_last_error(t0b_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int32_t t0b_is_poisoned(t0b_ctx* ctx) { return ctx && ctx->poisoned ? 1 : 0; }

int32_t t0b_num_sms(t0b_ctx* ctx) { return ctx ? ctx->num_sms : 0; }

int32_t t0b_set_sm_limit(t0b_ctx* ctx, int32_t sms) {
    if (!ctx) return T0B_ERR_INVALID;
    if (sms < 0 || sms > ctx->num_sms) return set_error(ctx, T0B_ERR_INVALID, "set_sm_limit: %d is outside 0..%d", sms, ctx->num_sms);
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    ctx->sm_limit = sms;
    return T0B_OK;
}

int32_t t0b_device_status(t0b_ctx* ctx, int32_t clear) {
    if (!ctx || !ctx->status_host) return 0;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    const int word = *reinterpret_cast<volatile int*>(ctx->status_host);
    const int st = word != 0 ? word : ctx->last_status;
    if (clear) {
        *reinterpret_cast<volatile int*>(ctx->status_host) = 0;
        ctx->last_status = 0;
    }
    return st;
}

int32_t t0b_set_wait_limit_ns(t0b_ctx* ctx, uint64_t ns) {
    if (!ctx || ns == 0) return T0B_ERR_INVALID;
    ctx->wait_limit_ns = ns;
    return T0B_OK;
}

int32_t t0b_alloc(t0b_ctx* ctx, size_t bytes, uint64_t* dptr) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (!dptr) return set_error(ctx, T0B_ERR_INVALID, "t0b_alloc: null out pointer");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    const size_t key = round4k(bytes == 0 ? 1 : bytes);
    auto it = ctx->pool_free.find(key);
    void* p = nullptr;
    if (it != ctx->pool_free.end()) {
        p = it->second;
        ctx->pool_free.erase(it);
        ctx->pool_cached -= key;
        ++ctx->pool_hits;
    } else {
        ++ctx->pool_misses;
        cudaError_t e = cudaMalloc(&p, key);
        if (e == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            // Give cached buffers back to the driver and retry once before reporting out-of-memory.
            for (auto& kv : ctx->pool_free) cudaFree(kv.second);
            ctx->pool_free.clear();
            ctx->pool_cached = 0;
            e = cudaMalloc(&p, key);
            if (e == cudaErrorMemoryAllocation) {
                cudaGetLastError();
                return set_error(ctx, T0B_ERR_NOMEM, "t0b_alloc: out of device memory for %zu bytes", key);
            }
        }
        if (e != cudaSuccess) return check_cuda(ctx, e, "cudaMalloc");
    }
    ctx->live[p] = key;
    *dptr = reinterpret_cast<uint64_t>(p);
    return T0B_OK;
}

int32_t t0b_alloc_zero(t0b_ctx* ctx, size_t bytes, uint64_t* dptr) {
    int32_t rc = t0b_alloc(ctx, bytes, dptr);
    if (rc != T0B_OK) return rc;
    return t0b_memset0(ctx, *dptr, bytes);
}

int32_t t0b_recycle(t0b_ctx* ctx, uint64_t dptr) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    void* p = reinterpret_cast<void*>(dptr);
    auto it = ctx->live.find(p);
    if (it == ctx->live.end()) return set_error(ctx, T0B_ERR_INVALID, "t0b_recycle: unknown buffer %p", p);
    drop_bf16_of(ctx, dptr);
    it = ctx->live.find(p);
    ctx->pool_free.emplace(it->second, p);
    ctx->pool_cached += it->second;
    ctx->live.erase(it);
    return T0B_OK;
}

int32_t t0b_free(t0b_ctx* ctx, uint64_t dptr) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    void* p = reinterpret_cast<void*>(dptr);
    auto it = ctx->live.find(p);
    if (it == ctx->live.end()) return set_error(ctx, T0B_ERR_INVALID, "t0b_free: unknown buffer %p", p);
    drop_bf16_of(ctx, dptr);
    ctx->live.erase(p);
    // Tensor maps that point into this buffer must not outlive it.
    ctx->tmaps.clear();
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaError_t e = cudaFree(p);
    if (e != cudaSuccess && !ctx->poisoned) return check_cuda(ctx, e, "cudaFree");
    return T0B_OK;
}

int32_t t0b_pool_stats(t0b_ctx* ctx, uint64_t* cached, uint64_t* hits, uint64_t* misses) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    if (cached) *cached = ctx->pool_cached;
    if (hits) *hits = ctx->pool_hits;
    if (misses) *misses = ctx->pool_misses;
    return T0B_OK;
}

int32_t t0b_memcpy_h2d(t0b_ctx* ctx, uint64_t dst, const void* src, size_t bytes) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (bytes == 0) return T0B_OK;
    if (!dst || !src) return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy_h2d: null pointer");
    {
        std::lock_guard<std::recursive_mutex> lk(ctx->mu);
        drop_bf16_of(ctx, dst);   // new contents: a cached bf16 copy of this buffer is stale
    }
    rc = check_cuda(ctx, cudaMemcpyAsync(reinterpret_cast<void*>(dst), src, bytes, cudaMemcpyHostToDevice, ctx->stream),
                    "cudaMemcpyAsync(h2d)");
    if (rc != T0B_OK) return rc;
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize(h2d)");
}

int32_t t0b_memcpy_d2h(t0b_ctx* ctx, void* dst, uint64_t src, size_t bytes) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (bytes == 0) return T0B_OK;
    if (!dst || !src) return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy_d2h: null pointer");
    rc = check_cuda(ctx, cudaMemcpyAsync(dst, reinterpret_cast<void*>(src), bytes, cudaMemcpyDeviceToHost, ctx->stream),
                    "cudaMemcpyAsync(d2h)");
    if (rc != T0B_OK) return rc;
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize(d2h)");
}

int32_t t0b_memcpy2d_d2h(t0b_ctx* ctx, void* dst, size_t dst_pitch, uint64_t src, size_t src_pitch, size_t width_bytes,
                         size_t height) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (width_bytes == 0 || height == 0) return T0B_OK;
    if (!dst || !src || dst_pitch < width_bytes || src_pitch < width_bytes)
        return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy2d_d2h: null pointer or pitch smaller than the row");
    rc = check_cuda(ctx, cudaMemcpy2DAsync(dst, dst_pitch, reinterpret_cast<void*>(src), src_pitch, width_bytes, height,
                                           cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpy2DAsync(d2h)");
    if (rc != T0B_OK) return rc;
    return check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize(d2h 2d)");
}

namespace {
// The copy streams of the asynchronous host copies and of the host-buffer GEMM, created on first use.
int32_t ensure_copy_streams(t0b_ctx* ctx) {
    if (ctx->h2d_stream) return T0B_OK;
    int32_t rc = check_cuda(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking), "cudaStreamCreate(h2d)");
    if (rc == T0B_OK) rc = check_cuda(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking), "cudaStreamCreate(d2h)");
    return rc;
}
// Make stream `later` wait for everything queued so far on stream `earlier`.
cudaError_t order_behind(cudaStream_t later, cudaStream_t earlier) {
    cudaEvent_t ev = nullptr;
    cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(ev, earlier);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(later, ev, 0);
    if (ev) cudaEventDestroy(ev);
    return e;
}
}  // namespace

int32_t t0b_memcpy_h2d_async(t0b_ctx* ctx, uint64_t dst, const void* src, size_t bytes) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (bytes == 0) return T0B_OK;
    if (!dst || !src) return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy_h2d_async: null pointer");
    if (ctx->capturing) return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy_h2d_async: not available during graph capture");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    drop_bf16_of(ctx, dst);
    rc = ensure_copy_streams(ctx);
    if (rc != T0B_OK) return rc;
    // The copy waits for the kernels queued so far (they may still read the destination) and later launches wait for it.
    cudaError_t e = order_behind(ctx->h2d_stream, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(reinterpret_cast<void*>(dst), src, bytes, cudaMemcpyHostToDevice, ctx->h2d_stream);
    if (e == cudaSuccess) e = order_behind(ctx->stream, ctx->h2d_stream);
    return check_cuda(ctx, e, "t0b_memcpy_h2d_async");
}

int32_t t0b_memcpy2d_d2h_async(t0b_ctx* ctx, void* dst, size_t dst_pitch, uint64_t src, size_t src_pitch, size_t width_bytes,
                               size_t height) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (width_bytes == 0 || height == 0) return T0B_OK;
    if (!dst || !src || dst_pitch < width_bytes || src_pitch < width_bytes)
        return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy2d_d2h_async: null pointer or pitch smaller than the row");
    if (ctx->capturing) return set_error(ctx, T0B_ERR_INVALID, "t0b_memcpy2d_d2h_async: not available during graph capture");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    rc = ensure_copy_streams(ctx);
    if (rc != T0B_OK) return rc;
    // Behind the work queued so far; launches made after this call do not wait for the copy.
    cudaError_t e = order_behind(ctx->d2h_stream, ctx->stream);
    if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(dst, dst_pitch, reinterpret_cast<void*>(src), src_pitch, width_bytes, height, cudaMemcpyDeviceToHost,
                              ctx->d2h_stream);
    ctx->d2h_pending = true;
    return check_cuda(ctx, e, "t0b_memcpy2d_d2h_async");
}

int32_t t0b_copy_d2d_async(t0b_ctx* ctx, uint64_t dst, size_t dst_pitch, uint64_t src, size_t src_pitch, size_t width_bytes,
                           size_t rows) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (width_bytes == 0 || rows == 0) return T0B_OK;
    if (!dst || !src || dst_pitch < width_bytes || src_pitch < width_bytes)
        return set_error(ctx, T0B_ERR_INVALID, "t0b_copy_d2d_async: null pointer or pitch smaller than the row");
    if (ctx->capturing) return set_error(ctx, T0B_ERR_INVALID, "t0b_copy_d2d_async: not available during graph capture");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    if (!ctx->p2p_stream) {
        rc = check_cuda(ctx, cudaStreamCreateWithFlags(&ctx->p2p_stream, cudaStreamNonBlocking), "cudaStreamCreate(p2p)");
        if (rc != T0B_OK) return rc;
    }
    // Behind the work queued so far on the compute stream; launches made after this call do not wait for the copy.
    cudaError_t e = order_behind(ctx->p2p_stream, ctx->stream);
    if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(reinterpret_cast<void*>(dst), dst_pitch, reinterpret_cast<void*>(src), src_pitch, width_bytes, rows,
                              cudaMemcpyDeviceToDevice, ctx->p2p_stream);
    ctx->p2p_pending = true;
    return check_cuda(ctx, e, "t0b_copy_d2d_async");
}

int32_t t0b_memset0(t0b_ctx* ctx, uint64_t dst, size_t bytes) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (bytes == 0) return T0B_OK;
    if (!dst) return set_error(ctx, T0B_ERR_INVALID, "t0b_memset0: null pointer");
    return check_cuda(ctx, cudaMemsetAsync(reinterpret_cast<void*>(dst), 0, bytes, ctx->stream), "cudaMemsetAsync");
}

int32_t t0b_sync(t0b_ctx* ctx) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    rc = check_cuda(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    if (rc != T0B_OK) return rc;
    if (ctx->p2p_pending) {   // side-stream device copies (t0b_copy_d2d_async) complete here too
        ctx->p2p_pending = false;
        rc = check_cuda(ctx, cudaStreamSynchronize(ctx->p2p_stream), "cudaStreamSynchronize(p2p)");
        if (rc != T0B_OK) return rc;
    }
    if (ctx->d2h_pending) {   // asynchronous read-backs (t0b_memcpy2d_d2h_async) complete here too
        ctx->d2h_pending = false;
        rc = check_cuda(ctx, cudaStreamSynchronize(ctx->d2h_stream), "cudaStreamSynchronize(d2h)");
        if (rc != T0B_OK) return rc;
    }
    const int st = take_device_status(ctx);
    if (st != 0) return set_error(ctx, T0B_ERR_DEVICE, "device status %d (101-105: a bounded in-kernel wait ran out; 110: an index outside its table)", st);
    return T0B_OK;
}

uint64_t t0b_launch_count(t0b_ctx* ctx) { return ctx ? ctx->launches : 0; }

// ------------------------------------------------------------------------------------------------ bf16 weight cache

int32_t t0b_get_or_create_bf16(t0b_ctx* ctx, uint64_t tensor_id, uint64_t f32_ptr, size_t n_elems, uint64_t* bf16_ptr) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (!bf16_ptr || !f32_ptr || n_elems == 0) return set_error(ctx, T0B_ERR_INVALID, "get_or_create_bf16: null pointer or no elements");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    auto it = ctx->bf16_cache.find(tensor_id);
    if (it != ctx->bf16_cache.end() && it->second.n == n_elems) {
        ++ctx->bf16_hits;
        *bf16_ptr = it->second.ptr;
        return T0B_OK;
    }
    if (it != ctx->bf16_cache.end()) {   // same id, another size: the old copy is stale
        t0b_recycle(ctx, it->second.ptr);
        ctx->bf16_cache.erase(it);
    }
    uint64_t out = 0;
    rc = t0b_alloc(ctx, ((n_elems * 2) + 255) & ~static_cast<size_t>(255), &out);
    if (rc != T0B_OK) return rc;
    rc = t0b_cast_f32_to_bf16(ctx, f32_ptr, out, n_elems, 1);   // stream-ordered before the GEMM that will read it
    if (rc != T0B_OK) {
        t0b_recycle(ctx, out);
        return rc;
    }
    ++ctx->bf16_conversions;
    ctx->bf16_cache[tensor_id] = t0b_ctx::Bf16Entry{out, n_elems};
    *bf16_ptr = out;
    return T0B_OK;
}

int32_t t0b_invalidate_bf16(t0b_ctx* ctx, uint64_t tensor_id) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    auto it = ctx->bf16_cache.find(tensor_id);
    if (it == ctx->bf16_cache.end()) return T0B_OK;
    t0b_recycle(ctx, it->second.ptr);   // reuse is stream-ordered behind the GEMMs that still read the copy
    ctx->bf16_cache.erase(it);
    return T0B_OK;
}

int32_t t0b_clear_bf16_cache(t0b_ctx* ctx) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    for (auto& kv : ctx->bf16_cache) t0b_recycle(ctx, kv.second.ptr);
    ctx->bf16_cache.clear();
    return T0B_OK;
}

int32_t t0b_bf16_cache_stats(t0b_ctx* ctx, uint64_t* entries, uint64_t* conversions, uint64_t* hits) {
    if (!ctx) return T0B_ERR_INVALID;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    if (entries) *entries = ctx->bf16_cache.size();
    if (conversions) *conversions = ctx->bf16_conversions;
    if (hits) *hits = ctx->bf16_hits;
    return T0B_OK;
}


// ------------------------------------------------------------------------------------------------ IPC

int32_t t0b_ipc_export(t0b_ctx* ctx, uint64_t dptr, uint8_t handle[64]) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (!dptr || !handle) return set_error(ctx, T0B_ERR_INVALID, "ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    rc = check_cuda(ctx, cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(dptr)), "cudaIpcGetMemHandle");
    if (rc != T0B_OK) return rc;
    std::memcpy(handle, &h, 64);
    return T0B_OK;
}

int32_t t0b_ipc_open(t0b_ctx* ctx, const uint8_t handle[64], uint64_t* dptr) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (!dptr || !handle) return set_error(ctx, T0B_ERR_INVALID, "ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void* p = nullptr;
    rc = check_cuda(ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    if (rc != T0B_OK) return rc;
    *dptr = reinterpret_cast<uint64_t>(p);
    return T0B_OK;
}

int32_t t0b_ipc_close(t0b_ctx* ctx, uint64_t dptr) {
    if (!ctx || !dptr) return T0B_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaError_t e = cudaIpcCloseMemHandle(reinterpret_cast<void*>(dptr));
    if (e != cudaSuccess && !ctx->poisoned) return check_cuda(ctx, e, "cudaIpcCloseMemHandle");
    return T0B_OK;
}

// ------------------------------------------------------------------------------------------------ graphs

int32_t t0b_graph_begin(t0b_ctx* ctx) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (ctx->capturing) return set_error(ctx, T0B_ERR_INVALID, "t0b_graph_begin: already capturing");
    rc = check_cuda(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    if (rc == T0B_OK) ctx->capturing = true;
    return rc;
}

int32_t t0b_graph_end(t0b_ctx* ctx, uint64_t* handle) {
    if (!ctx || !handle) return T0B_ERR_INVALID;
    if (!ctx->capturing) return set_error(ctx, T0B_ERR_INVALID, "t0b_graph_end: not capturing");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    int32_t rc = check_cuda(ctx, cudaStreamEndCapture(ctx->stream, &g), "cudaStreamEndCapture");
    if (rc != T0B_OK) return rc;
    cudaGraphExec_t ge = nullptr;
    rc = check_cuda(ctx, cudaGraphInstantiate(&ge, g, 0), "cudaGraphInstantiate");
    cudaGraphDestroy(g);
    if (rc != T0B_OK) return rc;
    const uint64_t id = ctx->next_graph++;
    ctx->graphs[id] = ge;
    *handle = id;
    return T0B_OK;
}

int32_t t0b_graph_launch(t0b_ctx* ctx, uint64_t handle, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    auto it = ctx->graphs.find(handle);
    if (it == ctx->graphs.end()) return set_error(ctx, T0B_ERR_INVALID, "t0b_graph_launch: unknown graph %llu",
                                                  static_cast<unsigned long long>(handle));
    rc = check_cuda(ctx, cudaGraphLaunch(it->second, ctx->stream), "cudaGraphLaunch");
    if (rc != T0B_OK) return rc;
    return finish(ctx, async, "graph launch");
}

int32_t t0b_graph_destroy(t0b_ctx* ctx, uint64_t handle) {
    if (!ctx) return T0B_ERR_INVALID;
    auto it = ctx->graphs.find(handle);
    if (it == ctx->graphs.end()) return T0B_ERR_INVALID;
    cudaGraphExecDestroy(it->second);
    ctx->graphs.erase(it);
    return T0B_OK;
}

}  // extern "C"
