// Embedding lookup and its gradient (src/t0/embedding_kernels.rs:30-96, src/ignis/ops/embedding.rs:25-178).
//   forward : out[t, :] = table[ids[t], :]                      (a gather: HBM-bound, 2 * tokens * dim * 4 bytes)
//   backward: grad_table[ids[t], :] += grad_out[t, :]           (a scatter-add)
// The reference's backward uses unordered global float atomics, so repeated ids make it non-reproducible.  Here the
// token positions are sorted by id first (stable radix sort of 32-bit keys, CUB), and one thread block per distinct id
// adds that id's gradient rows in ascending token order: the same order as the reference's CPU loop
// (embedding_kernels.rs:113-124), hence bit-identical to it, run after run, with every grad_out row read exactly once.
#include <cub/device/device_radix_sort.cuh>

#include <algorithm>

#include "t0b_internal.hpp"

using namespace t0b;

namespace {

constexpr int kThreads = 256;

// One block per token (grid-stride); VEC floats per thread per step.
template <int VEC>
__global__ void __launch_bounds__(kThreads) embedding_fwd_kernel(const float* __restrict__ table, const uint32_t* __restrict__ ids,
                                                                 float* __restrict__ out, uint32_t num_tokens, uint32_t dim,
                                                                 uint32_t vocab, int* status) {
    for (uint32_t t = blockIdx.x; t < num_tokens; t += gridDim.x) {
        const uint32_t id = ids[t];
        const bool ok = id < vocab;
        if (!ok && threadIdx.x == 0) *reinterpret_cast<volatile int*>(status) = kDevBadIndex;      // the row is written as zeros, nothing is read
        const float* src = table + static_cast<size_t>(ok ? id : 0) * dim;
        float* dst = out + static_cast<size_t>(t) * dim;
        if (VEC == 4) {
            for (uint32_t c = threadIdx.x * 4; c < dim; c += kThreads * 4) {
                const float4 v = ok ? __ldg(reinterpret_cast<const float4*>(src + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                __stcs(reinterpret_cast<float4*>(dst + c), v);
            }
        } else {
            for (uint32_t c = threadIdx.x; c < dim; c += kThreads) dst[c] = ok ? src[c] : 0.0f;
        }
    }
}

__global__ void iota_kernel(uint32_t* v, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) v[i] = i;
}

// Positions in the sorted id list where a new id starts, compacted in any order (each run is independent).
__global__ void segment_heads_kernel(const uint32_t* __restrict__ sorted_ids, uint32_t n, uint32_t* __restrict__ heads,
                                     uint32_t* __restrict__ n_heads) {
    for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < n; p += gridDim.x * blockDim.x)
        if (p == 0 || sorted_ids[p] != sorted_ids[p - 1]) heads[atomicAdd(n_heads, 1u)] = p;
}

// Work item = (run of equal ids, strip of kThreads * VEC columns).  The run's rows are added in sorted (= token)
// order; four rows are in flight at a time so the dependent adds do not serialise the loads.
template <int VEC>
__global__ void __launch_bounds__(kThreads) embedding_bwd_kernel(float* __restrict__ grad_table, const uint32_t* __restrict__ sorted_ids,
                                                                 const uint32_t* __restrict__ sorted_tok, const uint32_t* __restrict__ heads,
                                                                 const uint32_t* __restrict__ n_heads, const float* __restrict__ grad_out,
                                                                 uint32_t num_tokens, uint32_t dim, uint32_t vocab, int* status) {
    const uint32_t strips = (dim + kThreads * VEC - 1) / (kThreads * VEC);
    const uint64_t items = static_cast<uint64_t>(*n_heads) * strips;
    for (uint64_t item = blockIdx.x; item < items; item += gridDim.x) {
        const uint32_t p0 = heads[item / strips];
        const uint32_t strip = static_cast<uint32_t>(item % strips);
        const uint32_t id = sorted_ids[p0];
        if (id >= vocab) {
            if (threadIdx.x == 0) *reinterpret_cast<volatile int*>(status) = kDevBadIndex;         // skipped: nothing is written
            continue;
        }
        const uint32_t c = (strip * kThreads + threadIdx.x) * VEC;
        if (c >= dim) continue;
        float* dst = grad_table + static_cast<size_t>(id) * dim + c;
        float acc[VEC];
        if (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4*>(dst);
            acc[0] = v.x; acc[1] = v.y; acc[2] = v.z; acc[3] = v.w;
        } else {
            acc[0] = *dst;
        }
        uint32_t p = p0;
        while (p < num_tokens && sorted_ids[p] == id) {
            float g[4][VEC];
            int cnt = 0;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (p + u < num_tokens && sorted_ids[p + u] == id) {
                    const float* src = grad_out + static_cast<size_t>(sorted_tok[p + u]) * dim + c;
                    if (VEC == 4) {
                        const float4 v = __ldcs(reinterpret_cast<const float4*>(src));
                        g[u][0] = v.x; g[u][1] = v.y; g[u][2] = v.z; g[u][3] = v.w;
                    } else {
                        g[u][0] = __ldcs(src);
                    }
                    cnt = u + 1;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (u < cnt)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[e] += g[u][e];
            p += cnt;
        }
        if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        else *dst = acc[0];
    }
}

size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// Scratch layout of the backward: sorted ids | sorted token positions | token positions 0..n-1 | run heads | run count |
// radix-sort workspace.
struct BwdScratch {
    size_t sorted_ids, sorted_tok, iota, heads, n_heads, sort_tmp, sort_tmp_bytes, total;
};

int32_t bwd_scratch_layout(uint32_t num_tokens, BwdScratch* s) {
    size_t tmp = 0;
    const cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, tmp, static_cast<const uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                                          static_cast<const uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                                          static_cast<int>(num_tokens));
    if (e != cudaSuccess) return T0B_ERR_CUDA;
    const size_t arr = align256(static_cast<size_t>(num_tokens) * 4);
    s->sorted_ids = 0;
    s->sorted_tok = arr;
    s->iota = 2 * arr;
    s->heads = 3 * arr;
    s->n_heads = 4 * arr;
    s->sort_tmp = 4 * arr + 256;
    s->sort_tmp_bytes = tmp;
    s->total = s->sort_tmp + align256(tmp);
    return T0B_OK;
}

}  // namespace

extern "C" {

int32_t t0b_embedding_fwd(t0b_ctx* ctx, uint64_t table, uint64_t ids, uint64_t out, uint32_t num_tokens, uint32_t dim,
                          uint32_t vocab, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (num_tokens == 0 || dim == 0) return T0B_OK;
    if (!table || !ids || !out || vocab == 0) return set_error(ctx, T0B_ERR_INVALID, "embedding_fwd: null pointer or empty table");
    const int blocks = static_cast<int>(std::min<uint32_t>(num_tokens, static_cast<uint32_t>(ctx->num_sms) * 16));
    const bool vec = dim % 4 == 0 && table % 16 == 0 && out % 16 == 0;
    if (vec)
        embedding_fwd_kernel<4><<<blocks, kThreads, 0, ctx->stream>>>(reinterpret_cast<const float*>(table), reinterpret_cast<const uint32_t*>(ids),
                                                                      reinterpret_cast<float*>(out), num_tokens, dim, vocab, ctx->status_dev);
    else
        embedding_fwd_kernel<1><<<blocks, kThreads, 0, ctx->stream>>>(reinterpret_cast<const float*>(table), reinterpret_cast<const uint32_t*>(ids),
                                                                      reinterpret_cast<float*>(out), num_tokens, dim, vocab, ctx->status_dev);
    return finish(ctx, async, "embedding_fwd");
}

size_t t0b_embedding_bwd_scratch_bytes(uint32_t num_tokens) {
    BwdScratch s{};
    if (num_tokens == 0 || bwd_scratch_layout(num_tokens, &s) != T0B_OK) return 0;
    return s.total;
}

int32_t t0b_embedding_bwd(t0b_ctx* ctx, uint64_t grad_table, uint64_t ids, uint64_t grad_out, uint32_t num_tokens, uint32_t dim,
                          uint32_t vocab, uint64_t scratch, size_t scratch_bytes, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (num_tokens == 0 || dim == 0) return T0B_OK;
    if (!grad_table || !ids || !grad_out || vocab == 0)
        return set_error(ctx, T0B_ERR_INVALID, "embedding_bwd: null pointer or empty table");
    if (num_tokens > 0x7fffffffu) return set_error(ctx, T0B_ERR_INVALID, "embedding_bwd: more than 2^31-1 tokens");
    BwdScratch s{};
    if (bwd_scratch_layout(num_tokens, &s) != T0B_OK) return set_error(ctx, T0B_ERR_CUDA, "embedding_bwd: radix sort size query failed");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    uint64_t own = 0;
    if (!scratch) {
        rc = t0b_alloc(ctx, s.total, &own);        // from the pool; given back below, reuse is ordered by the stream
        if (rc != T0B_OK) return rc;
        scratch = own;
    } else if (scratch_bytes < s.total || scratch % 256 != 0) {
        return set_error(ctx, T0B_ERR_INVALID, "embedding_bwd: scratch must be 256-byte aligned and hold %zu bytes (got %zu)", s.total,
                         scratch_bytes);
    }
    auto at = [&](size_t off) { return reinterpret_cast<uint32_t*>(scratch + off); };
    const int lin_blocks = static_cast<int>(std::min<uint32_t>((num_tokens + 255) / 256, static_cast<uint32_t>(ctx->num_sms) * 8));
    int launched = 0;
    cudaError_t e = cudaMemsetAsync(at(s.n_heads), 0, 4, ctx->stream);
    if (e == cudaSuccess) {
        iota_kernel<<<lin_blocks, 256, 0, ctx->stream>>>(at(s.iota), num_tokens);
        ++launched;
        size_t tmp = s.sort_tmp_bytes;
        e = cub::DeviceRadixSort::SortPairs(reinterpret_cast<void*>(scratch + s.sort_tmp), tmp, reinterpret_cast<const uint32_t*>(ids),
                                            at(s.sorted_ids), at(s.iota), at(s.sorted_tok), static_cast<int>(num_tokens), 0, 32,
                                            ctx->stream);
    }
    if (e == cudaSuccess) {
        segment_heads_kernel<<<lin_blocks, 256, 0, ctx->stream>>>(at(s.sorted_ids), num_tokens, at(s.heads), at(s.n_heads));
        ++launched;
        const bool vec = dim % 4 == 0 && grad_table % 16 == 0 && grad_out % 16 == 0;
        const int blocks = ctx->num_sms * 8;
        if (vec)
            embedding_bwd_kernel<4><<<blocks, kThreads, 0, ctx->stream>>>(reinterpret_cast<float*>(grad_table), at(s.sorted_ids), at(s.sorted_tok),
                                                                          at(s.heads), at(s.n_heads), reinterpret_cast<const float*>(grad_out),
                                                                          num_tokens, dim, vocab, ctx->status_dev);
        else
            embedding_bwd_kernel<1><<<blocks, kThreads, 0, ctx->stream>>>(reinterpret_cast<float*>(grad_table), at(s.sorted_ids), at(s.sorted_tok),
                                                                          at(s.heads), at(s.n_heads), reinterpret_cast<const float*>(grad_out),
                                                                          num_tokens, dim, vocab, ctx->status_dev);
        ++launched;
    }
    if (own) t0b_recycle(ctx, own);
    if (e != cudaSuccess) return check_cuda(ctx, e, "embedding_bwd");
    return finish(ctx, async, "embedding_bwd", launched);
}

}  // extern "C"
