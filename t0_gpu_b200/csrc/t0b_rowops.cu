// Memory-bound kernels around the GEMMs: casts, RMSNorm, softmax, fused softmax cross-entropy, SiLU gate,
// gradient accumulate, AdamW.  All are HBM-bound: 128-bit accesses, one global read of each input where the
// row fits on chip, warp-shuffle + shared-memory block reductions, fixed reduction orders (no atomics).
// Reference kernels these stand in for: src/t0/rmsnorm_kernels.rs, src/ignis/ops/rmsnorm.rs,
// src/t0/softmax_kernels.rs, src/t0/ce_loss_kernels.rs, examples/kernels/softmax_ce_loss.rs,
// src/ignis/ops/silu.rs, src/t0/elementwise_kernels.rs, src/t0/adamw_kernels.rs.
#include <cuda_bf16.h>

#include <algorithm>
#include <cfloat>
#include <cstdlib>

#include "ptx_sm100.cuh"
#include <mutex>

#include "t0b_internal.hpp"

using namespace t0b;

namespace {

constexpr int kRowThreads = 512;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum of up to two values; every thread receives the totals.  `red` holds 2 * 32 floats.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();   // protect `red` against the previous use
    if (lane == 0) { red[warp] = a; red[32 + warp] = b; }
    __syncthreads();
    float x = lane < nwarps ? red[lane] : 0.0f;
    float y = lane < nwarps ? red[32 + lane] : 0.0f;
    a = warp_sum(x);
    b = warp_sum(y);
}

// Online softmax statistics (running max m, running sum s of exp(x - m)).  __expf (ex2.approx based, relative
// error ~1e-6) keeps these kernels memory-bound; the accurate expf made them instruction-bound.
__device__ __forceinline__ void online_add(float& m, float& s, float x) {
    if (x > m) { s = s * __expf(m - x) + 1.0f; m = x; }
    else s += __expf(x - m);
}
__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
    const float mm = fmaxf(m, m2);
    const float a = (m == -INFINITY) ? 0.0f : s * __expf(m - mm);
    const float b = (m2 == -INFINITY) ? 0.0f : s2 * __expf(m2 - mm);
    m = mm;
    s = a + b;
}
__device__ __forceinline__ void block_online(float& m, float& s, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        online_merge(m, s, m2, s2);
    }
    __syncthreads();
    if (lane == 0) { red[warp] = m; red[32 + warp] = s; }
    __syncthreads();
    m = lane < nwarps ? red[lane] : -INFINITY;
    s = lane < nwarps ? red[32 + lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        online_merge(m, s, m2, s2);
    }
}

// ------------------------------------------------------------------------------------------------ casts

__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                            size_t n) {
    ptx::grid_launch_dependents();
    const size_t n4 = n / 4;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0);
    size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (vec) {
        for (size_t j = i; j < n4; j += stride) {
            const float4 v = reinterpret_cast<const float4*>(src)[j];
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 o;
            o.x = *reinterpret_cast<uint32_t*>(&lo);
            o.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(dst)[j] = o;
        }
        for (size_t j = n4 * 4 + i; j < n; j += stride) dst[j] = __float2bfloat16_rn(src[j]);
    } else {
        for (size_t j = i; j < n; j += stride) dst[j] = __float2bfloat16_rn(src[j]);
    }
}

// src f32 [rows, cols] -> dst bf16 [cols, rows]; 32x32 tiles through shared memory, both sides coalesced.
__global__ void __launch_bounds__(256) cast_transpose_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                             uint32_t rows, uint32_t cols) {
    __shared__ float tile[32][33];
    const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (uint32_t j = ty; j < 32; j += 8) {
        const uint32_t r = r0 + j, c = c0 + tx;
        tile[j][tx] = (r < rows && c < cols) ? src[static_cast<size_t>(r) * cols + c] : 0.0f;
    }
    __syncthreads();
    for (uint32_t j = ty; j < 32; j += 8) {
        const uint32_t c = c0 + j, r = r0 + tx;
        if (r < rows && c < cols) dst[static_cast<size_t>(c) * rows + r] = __float2bfloat16_rn(tile[tx][j]);
    }
}

// ------------------------------------------------------------------------------------------------ RMSNorm

// One block per row.  The row is read once from HBM (second sweep hits L1/L2: a row is at most tens of KB).
__global__ void __launch_bounds__(kRowThreads) rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                  float* __restrict__ y, float* __restrict__ inv_rms,
                                                                  uint32_t cols, float eps) {
    __shared__ float red[64];
    const size_t row = blockIdx.x;
    const float* xr = x + row * cols;
    float* yr = y + row * cols;
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(y) & 15) == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    float ss = 0.0f, unused = 0.0f;
    if (vec) {
        for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) ss += xr[i] * xr[i];
    }
    block_sum2(ss, unused, red);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
    if (threadIdx.x == 0 && inv_rms) inv_rms[row] = rstd;
    if (vec) {
        for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            const float4 g = reinterpret_cast<const float4*>(w)[i];
            reinterpret_cast<float4*>(yr)[i] = make_float4(v.x * rstd * g.x, v.y * rstd * g.y, v.z * rstd * g.z, v.w * rstd * g.w);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) yr[i] = xr[i] * rstd * w[i];
    }
}

// Fast sigmoid (ex2.approx-based exponential and approximate reciprocal, relative error of a few 1e-7): the accurate
// expf and division made the fused RMSNorm+SiLU kernels instruction-bound.
__device__ __forceinline__ float sigmoidf_(float g) { return __fdividef(1.0f, 1.0f + __expf(-g)); }

__device__ __forceinline__ void silu_bwd_one(float gr, float g, float u, float& dgate, float& dup) {
    const float sig = sigmoidf_(g);
    dup = gr * g * sig;
    dgate = gr * u * sig * (1.0f + g * (1.0f - sig));
}

__device__ __forceinline__ uint2 pack_bf16x4(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    return o;
}

// Register-resident forward for rows of up to 4 * VPT * blockDim.x columns: CTAs walk rows with a grid stride,
// the weight stays in registers for all of them and each row's x is read exactly once.
// SILU16: the row is passed through SiLU and stored as bf16 (the input of the next GEMM) -- the values the
// three-kernel sequence RMSNorm, SiLU, f32->bf16 cast would store, without the two f32 round trips through HBM.
template <int VPT, bool SILU16 = false>
__global__ void __launch_bounds__(kRowThreads, VPT <= 2 ? 4 : 1) rmsnorm_fwd_reg_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                      void* __restrict__ y, float* __restrict__ inv_rms,
                                                                      uint32_t rows, uint32_t cols, float eps) {
    ptx::grid_launch_dependents();
    __shared__ float red[64];
    const uint32_t n4 = cols / 4;
    float4 wv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        wv[j] = i < n4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(row) * cols);
        float4* yr = reinterpret_cast<float4*>(static_cast<float*>(y) + static_cast<size_t>(row) * cols);
        uint2* yh = reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(y) + static_cast<size_t>(row) * cols);
        float4 xv[VPT];
        float ss = 0.0f, unused = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            xv[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
        }
        block_sum2(ss, unused, red);
        const float rstd = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
        if (threadIdx.x == 0 && inv_rms) inv_rms[row] = rstd;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            if (i >= n4) continue;
            const float4 r = make_float4(xv[j].x * rstd * wv[j].x, xv[j].y * rstd * wv[j].y, xv[j].z * rstd * wv[j].z,
                                         xv[j].w * rstd * wv[j].w);
            if (SILU16) yh[i] = pack_bf16x4(r.x * sigmoidf_(r.x), r.y * sigmoidf_(r.y), r.z * sigmoidf_(r.z), r.w * sigmoidf_(r.w));
            else yr[i] = r;
        }
    }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(x * dy*w)); also stores rstd per row for the dgamma stage.
__global__ void __launch_bounds__(kRowThreads) rmsnorm_bwd_dx_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                     const float* __restrict__ w, float* __restrict__ dx,
                                                                     float* __restrict__ inv_rms, uint32_t cols, float eps) {
    __shared__ float red[64];
    const size_t row = blockIdx.x;
    const float* xr = x + row * cols;
    const float* dyr = dy + row * cols;
    float* dxr = dx ? dx + row * cols : nullptr;
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(dy) & 15) == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(dx) & 15) == 0);
    float ss = 0.0f, dot = 0.0f;
    if (vec) {
        for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            const float4 d = reinterpret_cast<const float4*>(dyr)[i];
            const float4 g = reinterpret_cast<const float4*>(w)[i];
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            dot += v.x * d.x * g.x + v.y * d.y * g.y + v.z * d.z * g.z + v.w * d.w * g.w;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
            ss += xr[i] * xr[i];
            dot += xr[i] * dyr[i] * w[i];
        }
    }
    block_sum2(ss, dot, red);
    const float rstd = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
    const float coef = rstd * rstd * (dot / static_cast<float>(cols));
    if (threadIdx.x == 0 && inv_rms) inv_rms[row] = rstd;
    if (!dxr) return;
    if (vec) {
        for (uint32_t i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(xr)[i];
            const float4 d = reinterpret_cast<const float4*>(dyr)[i];
            const float4 g = reinterpret_cast<const float4*>(w)[i];
            reinterpret_cast<float4*>(dxr)[i] =
                make_float4(rstd * (d.x * g.x - v.x * coef), rstd * (d.y * g.y - v.y * coef),
                            rstd * (d.z * g.z - v.z * coef), rstd * (d.w * g.w - v.w * coef));
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) dxr[i] = rstd * (dyr[i] * w[i] - xr[i] * coef);
    }
}

// dgamma stage 1: block (cb, rb) sums dy*x*inv_rms over its row range, rows ascending, one column per thread.
__global__ void __launch_bounds__(256) rmsnorm_dgamma_partial_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                     const float* __restrict__ inv_rms,
                                                                     float* __restrict__ partial, uint32_t rows,
                                                                     uint32_t cols, uint32_t rows_per_block) {
    const uint32_t c = blockIdx.x * 256 + threadIdx.x;
    const uint32_t r0 = blockIdx.y * rows_per_block;
    const uint32_t r1 = min(rows, r0 + rows_per_block);
    if (c >= cols) return;
    float acc = 0.0f;
    for (uint32_t r = r0; r < r1; ++r) {
        const size_t i = static_cast<size_t>(r) * cols + c;
        acc += dy[i] * x[i] * inv_rms[r];
    }
    partial[static_cast<size_t>(blockIdx.y) * cols + c] = acc;
}
// dgamma stage 2: sum the row-block partials in a fixed order.  A block owns 32 columns; its 8 warps each add every
// 8th partial row (ascending), then warp 0 adds the 8 sums in warp order.  Launch with kDgammaFinalGrid(cols) blocks.
__global__ void __launch_bounds__(256) rmsnorm_dgamma_final_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                                                   uint32_t cols, uint32_t nblocks) {
    ptx::grid_launch_dependents();
    __shared__ float part[8][32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t c = blockIdx.x * 32 + lane;
    float acc = 0.0f;
    if (c < cols) {
#pragma unroll 4
        for (uint32_t b = warp; b < nblocks; b += 8) acc += partial[static_cast<size_t>(b) * cols + c];
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && c < cols) {
        float total = part[0][lane];
#pragma unroll
        for (int w = 1; w < 8; ++w) total += part[w][lane];
        dgamma[c] = total;
    }
}
inline uint32_t kDgammaFinalGrid(uint32_t cols) { return (cols + 31) / 32; }

constexpr uint32_t kDgammaRowBlocks = 64;

// Fused RMSNorm backward: each CTA walks rows r = blockIdx.x, blockIdx.x + gridDim.x, ... keeping the row's x and
// dy in registers between the reduction sweep and the dx sweep (one HBM read of each), and accumulates its share of
// dgamma[c] = sum_r dy*x*rstd in registers; per-CTA partials are then summed in CTA order by
// rmsnorm_dgamma_final_kernel.  Every thread owns VPT float4 column groups: cols <= 4 * VPT * blockDim.x.
// SILU16: dy is the gradient of SiLU(RMSNorm(x)); the normalised row is recomputed from x, the SiLU derivative is
// applied in registers and dx is stored as bf16 -- the values of the sequence SiLU backward, RMSNorm backward, cast.
template <int VPT, bool SILU16 = false>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_bwd_fused_kernel(const float* __restrict__ dy, const float* __restrict__ x,
                                                                        const float* __restrict__ w, void* __restrict__ dx,
                                                                        float* __restrict__ partial, uint32_t rows,
                                                                        uint32_t cols, float eps) {
    ptx::grid_launch_dependents();
    __shared__ float red[64];
    const uint32_t n4 = cols / 4;
    float4 wv[VPT], acc[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        wv[j] = i < n4 ? reinterpret_cast<const float4*>(w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* xr = reinterpret_cast<const float4*>(x + static_cast<size_t>(row) * cols);
        const float4* dyr = reinterpret_cast<const float4*>(dy + static_cast<size_t>(row) * cols);
        float4 xv[VPT], dv[VPT];
        float ss = 0.0f, dot = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            if (i < n4) {
                xv[j] = xr[i];
                dv[j] = dyr[i];
            } else {
                xv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                dv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            ss += xv[j].x * xv[j].x + xv[j].y * xv[j].y + xv[j].z * xv[j].z + xv[j].w * xv[j].w;
            if (!SILU16)
                dot += xv[j].x * dv[j].x * wv[j].x + xv[j].y * dv[j].y * wv[j].y + xv[j].z * dv[j].z * wv[j].z + xv[j].w * dv[j].w * wv[j].w;
        }
        float rstd;
        if (SILU16) {
            float unused = 0.0f;
            block_sum2(ss, unused, red);
            rstd = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                float du;
                silu_bwd_one(dv[j].x, xv[j].x * rstd * wv[j].x, 1.0f, dv[j].x, du);
                silu_bwd_one(dv[j].y, xv[j].y * rstd * wv[j].y, 1.0f, dv[j].y, du);
                silu_bwd_one(dv[j].z, xv[j].z * rstd * wv[j].z, 1.0f, dv[j].z, du);
                silu_bwd_one(dv[j].w, xv[j].w * rstd * wv[j].w, 1.0f, dv[j].w, du);
                dot += xv[j].x * dv[j].x * wv[j].x + xv[j].y * dv[j].y * wv[j].y + xv[j].z * dv[j].z * wv[j].z + xv[j].w * dv[j].w * wv[j].w;
            }
            unused = 0.0f;
            block_sum2(dot, unused, red);
        } else {
            block_sum2(ss, dot, red);
            rstd = 1.0f / sqrtf(ss / static_cast<float>(cols) + eps);
        }
        const float coef = rstd * rstd * (dot / static_cast<float>(cols));
        float4* dxr = (dx && !SILU16) ? reinterpret_cast<float4*>(static_cast<float*>(dx) + static_cast<size_t>(row) * cols) : nullptr;
        uint2* dxh = (dx && SILU16) ? reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(dx) + static_cast<size_t>(row) * cols) : nullptr;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            acc[j].x += dv[j].x * xv[j].x * rstd;
            acc[j].y += dv[j].y * xv[j].y * rstd;
            acc[j].z += dv[j].z * xv[j].z * rstd;
            acc[j].w += dv[j].w * xv[j].w * rstd;
            if (i >= n4) continue;
            const float4 o = make_float4(rstd * (dv[j].x * wv[j].x - xv[j].x * coef), rstd * (dv[j].y * wv[j].y - xv[j].y * coef),
                                         rstd * (dv[j].z * wv[j].z - xv[j].z * coef), rstd * (dv[j].w * wv[j].w - xv[j].w * coef));
            if (dxr) dxr[i] = o;
            if (dxh) dxh[i] = pack_bf16x4(o.x, o.y, o.z, o.w);
        }
    }
    if (partial == nullptr) return;   // dx only
    float4* pr = reinterpret_cast<float4*>(partial + static_cast<size_t>(blockIdx.x) * cols);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        if (i < n4) pr[i] = acc[j];
    }
}

__host__ __device__ inline uint32_t rmsnorm_fused_ctas(uint32_t rows) {
    uint32_t g = rows / 4;
    if (g < 1) g = 1;
    if (g > 512) g = 512;
    return g;
}


// ------------------------------------------------------------------------------------------------ softmax / CE

// Row statistics with the row cached in shared memory when it fits (one HBM read), else re-read.
template <bool CACHE>
__device__ __forceinline__ void row_stats(const float* __restrict__ xr, uint32_t cols, float* cache, float* red, float& m,
                                          float& s) {
    m = -INFINITY;
    s = 0.0f;
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
    if (vec) {
        // Four independent 16-byte loads in flight per thread before the dependent max/sum update.
        const uint32_t n4 = cols / 4;
        for (uint32_t i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                v[u] = i < n4 ? reinterpret_cast<const float4*>(xr)[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                if (i < n4) {
                    if (CACHE) reinterpret_cast<float4*>(cache)[i] = v[u];
                    const float lm = fmaxf(fmaxf(v[u].x, v[u].y), fmaxf(v[u].z, v[u].w));
                    if (lm > m) { s *= __expf(m - lm); m = lm; }
                    s += __expf(v[u].x - m) + __expf(v[u].y - m) + __expf(v[u].z - m) + __expf(v[u].w - m);
                }
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = xr[i];
            if (CACHE) cache[i] = v;
            online_add(m, s, v);
        }
    }
    block_online(m, s, red);
}

template <bool CACHE>
__global__ void __launch_bounds__(kRowThreads) softmax_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                  uint32_t cols) {
    extern __shared__ __align__(16) float cache[];
    __shared__ float red[64];
    const size_t row = blockIdx.x;
    const float* xr = x + row * cols;
    float* yr = y + row * cols;
    float m, s;
    row_stats<CACHE>(xr, cols, cache, red, m, s);
    const float inv = 1.0f / s;
    const float* src = CACHE ? cache : xr;
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) && ((reinterpret_cast<uintptr_t>(yr) & 15) == 0);
    if (vec) {
        const uint32_t n4 = cols / 4;
        for (uint32_t i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                if (i < n4) v[u] = reinterpret_cast<const float4*>(src)[i];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                if (i < n4)
                    reinterpret_cast<float4*>(yr)[i] = make_float4(__expf(v[u].x - m) * inv, __expf(v[u].y - m) * inv,
                                                                   __expf(v[u].z - m) * inv, __expf(v[u].w - m) * inv);
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) yr[i] = __expf(src[i] - m) * inv;
    }
}

__global__ void __launch_bounds__(kRowThreads) softmax_bwd_kernel(const float* __restrict__ dy, const float* __restrict__ y,
                                                                  float* __restrict__ dx, uint32_t cols) {
    __shared__ float red[64];
    const size_t row = blockIdx.x;
    const float* dyr = dy + row * cols;
    const float* yr = y + row * cols;
    float* dxr = dx + row * cols;
    float dot = 0.0f, unused = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) dot += dyr[i] * yr[i];
    block_sum2(dot, unused, red);
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) dxr[i] = yr[i] * (dyr[i] - dot);
}

// Fused softmax cross-entropy over one row per block: loss = log(sum exp(x - max)) + max - x[target];
// dlogits = (exp(x - max) / sum - onehot) * scale.
// GRAD16: the gradient is stored as bf16 (round to nearest even of the same f32 values), ready to be a GEMM operand.
template <bool CACHE, bool GRAD16 = false>
__global__ void __launch_bounds__(kRowThreads) softmax_ce_kernel(const float* __restrict__ logits,
                                                                 const uint32_t* __restrict__ targets,
                                                                 float* __restrict__ losses, void* __restrict__ dlogits,
                                                                 uint32_t cols, size_t ld, float scale) {
    ptx::grid_launch_dependents();
    extern __shared__ __align__(16) float cache[];
    __shared__ float red[64];
    const size_t row = blockIdx.x;
    const float* xr = logits + row * ld;
    float m, s;
    row_stats<CACHE>(xr, cols, cache, red, m, s);
    const uint32_t t = targets[row];
    if (threadIdx.x == 0 && losses) losses[row] = (t < cols) ? (logf(s) + m - xr[t]) : 0.0f;
    if (!dlogits) return;
    float* dr = static_cast<float*>(dlogits) + row * ld;
    __nv_bfloat16* dh = static_cast<__nv_bfloat16*>(dlogits) + row * ld;
    const float inv = 1.0f / s;
    const float* src = CACHE ? cache : xr;
    const bool vec = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) &&
                     (GRAD16 ? (reinterpret_cast<uintptr_t>(dh) & 7) == 0 : (reinterpret_cast<uintptr_t>(dr) & 15) == 0);
    if (vec) {
        const uint32_t n4 = cols / 4;
        for (uint32_t i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                if (i < n4) v[u] = reinterpret_cast<const float4*>(src)[i];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                if (i >= n4) continue;
                float4 o = make_float4(__expf(v[u].x - m) * inv, __expf(v[u].y - m) * inv, __expf(v[u].z - m) * inv,
                                       __expf(v[u].w - m) * inv);
                const uint32_t c = i * 4;
                if (t - c < 4u) {
                    if (t == c) o.x -= 1.0f;
                    else if (t == c + 1) o.y -= 1.0f;
                    else if (t == c + 2) o.z -= 1.0f;
                    else o.w -= 1.0f;
                }
                if (GRAD16) reinterpret_cast<uint2*>(dh)[i] = pack_bf16x4(o.x * scale, o.y * scale, o.z * scale, o.w * scale);
                else reinterpret_cast<float4*>(dr)[i] = make_float4(o.x * scale, o.y * scale, o.z * scale, o.w * scale);
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
            const float g = (__expf(src[i] - m) * inv - (i == t ? 1.0f : 0.0f)) * scale;
            if (GRAD16) dh[i] = __float2bfloat16_rn(g);
            else dr[i] = g;
        }
    }
}

// ------------------------------------------------------------------------------------------------ element-wise

__global__ void __launch_bounds__(256) silu_gate_fwd_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                            float* __restrict__ out, size_t n) {
    ptx::grid_launch_dependents();
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(gate) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                     (!up || (reinterpret_cast<uintptr_t>(up) & 15) == 0);
    size_t done = 0;
    if (vec) {
        const size_t n4 = n / 4;
        for (size_t i = i0; i < n4; i += stride) {
            const float4 g = reinterpret_cast<const float4*>(gate)[i];
            float4 u = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            if (up) u = reinterpret_cast<const float4*>(up)[i];
            reinterpret_cast<float4*>(out)[i] = make_float4(g.x * sigmoidf_(g.x) * u.x, g.y * sigmoidf_(g.y) * u.y,
                                                            g.z * sigmoidf_(g.z) * u.z, g.w * sigmoidf_(g.w) * u.w);
        }
        done = n4 * 4;
    }
    for (size_t i = done + i0; i < n; i += stride) {
        const float g = gate[i];
        out[i] = g * sigmoidf_(g) * (up ? up[i] : 1.0f);
    }
}

__global__ void __launch_bounds__(256) silu_gate_bwd_kernel(const float* __restrict__ grad, const float* __restrict__ gate,
                                                            const float* __restrict__ up, float* __restrict__ dgate,
                                                            float* __restrict__ dup, size_t n) {
    ptx::grid_launch_dependents();
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(grad) & 15) == 0) && ((reinterpret_cast<uintptr_t>(gate) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(dgate) & 15) == 0) && (!up || (reinterpret_cast<uintptr_t>(up) & 15) == 0) &&
                     (!dup || (reinterpret_cast<uintptr_t>(dup) & 15) == 0);
    size_t done = 0;
    if (vec) {
        const size_t n4 = n / 4;
        for (size_t i = i0; i < n4; i += stride) {
            const float4 gr = reinterpret_cast<const float4*>(grad)[i];
            const float4 g = reinterpret_cast<const float4*>(gate)[i];
            float4 u = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            if (up) u = reinterpret_cast<const float4*>(up)[i];
            float4 dg, du;
            silu_bwd_one(gr.x, g.x, u.x, dg.x, du.x);
            silu_bwd_one(gr.y, g.y, u.y, dg.y, du.y);
            silu_bwd_one(gr.z, g.z, u.z, dg.z, du.z);
            silu_bwd_one(gr.w, g.w, u.w, dg.w, du.w);
            reinterpret_cast<float4*>(dgate)[i] = dg;
            if (dup) reinterpret_cast<float4*>(dup)[i] = du;
        }
        done = n4 * 4;
    }
    for (size_t i = done + i0; i < n; i += stride) {
        float dg, du;
        silu_bwd_one(grad[i], gate[i], up ? up[i] : 1.0f, dg, du);
        dgate[i] = dg;
        if (dup) dup[i] = du;
    }
}

__global__ void __launch_bounds__(256) residual_add_kernel(float* __restrict__ y, const float* __restrict__ x, size_t n) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(y) & 15) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (vec) {
        const size_t n4 = n / 4;
        for (size_t i = i0; i < n4; i += stride) {
            float4 a = reinterpret_cast<float4*>(y)[i];
            const float4 b = reinterpret_cast<const float4*>(x)[i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            reinterpret_cast<float4*>(y)[i] = a;
        }
        for (size_t i = n4 * 4 + i0; i < n; i += stride) y[i] += x[i];
    } else {
        for (size_t i = i0; i < n; i += stride) y[i] += x[i];
    }
}

__device__ __forceinline__ float adamw_one(float p, float gi, float& m, float& v, float lr, float beta1, float beta2,
                                           float eps, float wd, float bc1, float bc2) {
    m = beta1 * m + (1.0f - beta1) * gi;
    v = beta2 * v + (1.0f - beta2) * gi * gi;
    return p * (1.0f - lr * wd) - lr * (m * bc1) / (sqrtf(v * bc2) + eps);
}

__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                    float* __restrict__ v, __nv_bfloat16* __restrict__ p_bf16, size_t n,
                                                    float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                                    float bc2, float grad_scale) {
    ptx::grid_launch_dependents();
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const bool vec = (((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                        reinterpret_cast<uintptr_t>(v)) & 15) == 0) && ((reinterpret_cast<uintptr_t>(p_bf16) & 7) == 0);
    size_t done = 0;
    if (vec) {
        const size_t n4 = n / 4;
        for (size_t i = i0; i < n4; i += stride) {
            float4 pp = reinterpret_cast<float4*>(p)[i];
            const float4 gg = reinterpret_cast<const float4*>(g)[i];
            float4 mm = reinterpret_cast<float4*>(m)[i];
            float4 vv = reinterpret_cast<float4*>(v)[i];
            pp.x = adamw_one(pp.x, gg.x * grad_scale, mm.x, vv.x, lr, beta1, beta2, eps, wd, bc1, bc2);
            pp.y = adamw_one(pp.y, gg.y * grad_scale, mm.y, vv.y, lr, beta1, beta2, eps, wd, bc1, bc2);
            pp.z = adamw_one(pp.z, gg.z * grad_scale, mm.z, vv.z, lr, beta1, beta2, eps, wd, bc1, bc2);
            pp.w = adamw_one(pp.w, gg.w * grad_scale, mm.w, vv.w, lr, beta1, beta2, eps, wd, bc1, bc2);
            reinterpret_cast<float4*>(p)[i] = pp;
            reinterpret_cast<float4*>(m)[i] = mm;
            reinterpret_cast<float4*>(v)[i] = vv;
            if (p_bf16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
                uint2 o;
                o.x = *reinterpret_cast<uint32_t*>(&lo);
                o.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(p_bf16)[i] = o;
            }
        }
        done = n4 * 4;
    }
    for (size_t i = done + i0; i < n; i += stride) {
        float mi = m[i], vi = v[i];
        const float pn = adamw_one(p[i], g[i] * grad_scale, mi, vi, lr, beta1, beta2, eps, wd, bc1, bc2);
        m[i] = mi;
        v[i] = vi;
        p[i] = pn;
        if (p_bf16) p_bf16[i] = __float2bfloat16_rn(pn);
    }
}

int grid_for(t0b_ctx* ctx, size_t n, int per_block) {
    const size_t blocks = (n + per_block - 1) / per_block;
    return static_cast<int>(std::max<size_t>(1, std::min<size_t>(blocks, static_cast<size_t>(ctx->num_sms) * 16)));
}

// Rows up to 64 KiB are cached in shared memory (several CTAs still fit per SM, one HBM read); wider rows are
// re-read through L2 instead, which measured faster than one 128 KiB-row CTA per SM.
constexpr size_t kRowCacheLimit = 200 * 1024;
constexpr size_t kRowCacheMax = 64 * 1024;

}  // namespace

extern "C" {

int32_t t0b_cast_f32_to_bf16(t0b_ctx* ctx, uint64_t src, uint64_t dst, size_t n, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (n == 0) return T0B_OK;
    if (!src || !dst) return set_error(ctx, T0B_ERR_INVALID, "cast: null pointer");
    cast_f32_bf16_kernel<<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>(reinterpret_cast<const float*>(src),
                                                                              reinterpret_cast<__nv_bfloat16*>(dst), n);
    return finish(ctx, async, "cast_f32_to_bf16");
}

int32_t t0b_cast_f32_to_bf16_transpose(t0b_ctx* ctx, uint64_t src, uint64_t dst, uint32_t rows, uint32_t cols,
                                       int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0 || cols == 0) return T0B_OK;
    if (!src || !dst) return set_error(ctx, T0B_ERR_INVALID, "cast_transpose: null pointer");
    dim3 grid((cols + 31) / 32, (rows + 31) / 32);
    if (grid.y > 65535) return set_error(ctx, T0B_ERR_INVALID, "cast_transpose: too many rows (%u)", rows);
    cast_transpose_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float*>(src),
                                                         reinterpret_cast<__nv_bfloat16*>(dst), rows, cols);
    return finish(ctx, async, "cast_f32_to_bf16_transpose");
}

int32_t t0b_rmsnorm_fwd(t0b_ctx* ctx, uint64_t x, uint64_t weight, uint64_t y, uint64_t inv_rms, uint32_t rows,
                        uint32_t cols, float eps, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) return T0B_OK;
    if (cols == 0 || !x || !weight || !y) return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_fwd: null pointer or zero cols");
    const int threads = cols >= 2048 ? kRowThreads : (cols >= 512 ? 128 : 32);
    if (((x | weight | y) & 15) == 0 && cols % 4 == 0 && cols >= 1024 && cols <= 4u * 4u * kRowThreads) {
        const uint32_t g = std::min<uint32_t>(rows, static_cast<uint32_t>(ctx->num_sms) * 4u);
        const uint32_t n4 = cols / 4;
        const float* xp = reinterpret_cast<const float*>(x);
        const float* wp = reinterpret_cast<const float*>(weight);
        float* yp = reinterpret_cast<float*>(y);
        float* ip = reinterpret_cast<float*>(inv_rms);
        if (n4 <= 1u * kRowThreads) rmsnorm_fwd_reg_kernel<1><<<g, kRowThreads, 0, ctx->stream>>>(xp, wp, yp, ip, rows, cols, eps);
        else if (n4 <= 2u * kRowThreads) rmsnorm_fwd_reg_kernel<2><<<g, kRowThreads, 0, ctx->stream>>>(xp, wp, yp, ip, rows, cols, eps);
        else rmsnorm_fwd_reg_kernel<4><<<g, kRowThreads, 0, ctx->stream>>>(xp, wp, yp, ip, rows, cols, eps);
        return finish(ctx, async, "rmsnorm_fwd");
    }
    rmsnorm_fwd_kernel<<<rows, threads, 0, ctx->stream>>>(reinterpret_cast<const float*>(x), reinterpret_cast<const float*>(weight),
                                                          reinterpret_cast<float*>(y), reinterpret_cast<float*>(inv_rms), cols, eps);
    return finish(ctx, async, "rmsnorm_fwd");
}

size_t t0b_rmsnorm_bwd_scratch_bytes(uint32_t rows, uint32_t cols) {
    const size_t blocks = std::max<size_t>(kDgammaRowBlocks, rmsnorm_fused_ctas(rows));
    return (((static_cast<size_t>(rows) + 3) & ~static_cast<size_t>(3)) + blocks * cols) * sizeof(float);
}

int32_t t0b_rmsnorm_bwd(t0b_ctx* ctx, uint64_t dy, uint64_t x, uint64_t weight, uint64_t dx, uint64_t dgamma,
                        uint64_t scratch, size_t scratch_bytes, uint32_t rows, uint32_t cols, float eps, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) {
        if (dgamma && cols) return t0b_memset0(ctx, dgamma, static_cast<size_t>(cols) * 4);
        return T0B_OK;
    }
    if (cols == 0 || !dy || !x || !weight || (!dx && !dgamma)) return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_bwd: null pointer or zero cols");
    float* inv = nullptr;
    float* partial = nullptr;
    if (dgamma) {
        if (!scratch || scratch_bytes < t0b_rmsnorm_bwd_scratch_bytes(rows, cols))
            return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_bwd: dgamma needs %zu bytes of scratch, got %zu",
                             t0b_rmsnorm_bwd_scratch_bytes(rows, cols), scratch_bytes);
        inv = reinterpret_cast<float*>(scratch);
        partial = inv + rows;
    }
    const int threads = cols >= 2048 ? kRowThreads : (cols >= 512 ? 128 : 32);
    const bool aligned = ((dy | x | weight | dx | scratch) & 15) == 0 && cols % 4 == 0;
    if (aligned && cols >= 1024 && cols <= 4u * 4u * kRowThreads) {
        // One pass over dy and x: dx and the per-CTA dgamma partials come out of the same kernel.
        const uint32_t g = dgamma ? rmsnorm_fused_ctas(rows) : std::min<uint32_t>(rows, static_cast<uint32_t>(ctx->num_sms) * 4u);
        const uint32_t n4 = cols / 4;
        if (dgamma) partial = reinterpret_cast<float*>(scratch) + ((static_cast<size_t>(rows) + 3) & ~static_cast<size_t>(3));   // 16-byte aligned
        if (n4 <= 1u * kRowThreads)
            rmsnorm_bwd_fused_kernel<1><<<g, kRowThreads, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                reinterpret_cast<const float*>(weight), reinterpret_cast<float*>(dx), partial, rows, cols, eps);
        else if (n4 <= 2u * kRowThreads)
            rmsnorm_bwd_fused_kernel<2><<<g, kRowThreads, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                reinterpret_cast<const float*>(weight), reinterpret_cast<float*>(dx), partial, rows, cols, eps);
        else
            rmsnorm_bwd_fused_kernel<4><<<g, kRowThreads, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                reinterpret_cast<const float*>(weight), reinterpret_cast<float*>(dx), partial, rows, cols, eps);
        rc = check_cuda(ctx, cudaGetLastError(), "rmsnorm_bwd_fused launch");
        if (rc != T0B_OK) return rc;
        if (dgamma) {
            ++ctx->launches;
            rmsnorm_dgamma_final_kernel<<<kDgammaFinalGrid(cols), 256, 0, ctx->stream>>>(partial, reinterpret_cast<float*>(dgamma), cols, g);
        }
        return finish(ctx, async, "rmsnorm_bwd");
    }
    rmsnorm_bwd_dx_kernel<<<rows, threads, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                                                             reinterpret_cast<const float*>(weight), reinterpret_cast<float*>(dx),
                                                             inv, cols, eps);
    rc = check_cuda(ctx, cudaGetLastError(), "rmsnorm_bwd_dx launch");
    if (rc != T0B_OK) return rc;
    if (dgamma) {
        ++ctx->launches;
        const uint32_t nblocks = std::min(kDgammaRowBlocks, rows);
        const uint32_t rpb = (rows + nblocks - 1) / nblocks;
        const uint32_t used = (rows + rpb - 1) / rpb;
        dim3 grid((cols + 255) / 256, used);
        rmsnorm_dgamma_partial_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                                                                     inv, partial, rows, cols, rpb);
        rc = check_cuda(ctx, cudaGetLastError(), "rmsnorm_dgamma_partial launch");
        if (rc != T0B_OK) return rc;
        ++ctx->launches;
        rmsnorm_dgamma_final_kernel<<<kDgammaFinalGrid(cols), 256, 0, ctx->stream>>>(partial, reinterpret_cast<float*>(dgamma), cols, used);
    }
    return finish(ctx, async, "rmsnorm_bwd");
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that cannot allocate device memory.
//
// Some users of this library own no allocator they may call at this point: a host runtime that reserved its
// whole device budget at start-up and hands out fixed buffers only (the reference's runtime keeps such a VRAM
// pool), or a training loop that must not hit the device-wide synchronisation cudaMalloc / cudaFree imply in
// the middle of a step.  They can pass inputs and outputs, but have nowhere to get the dgamma scratch from.
// This entry point keeps that scratch inside the library image instead: a fixed array in device global
// memory, 2 MiB, present on every GPU that loads the library until the process exits.
//
// The array's name is only a host-side stand-in for the symbol; the device address is looked up with
// cudaGetSymbolAddress, once per device, with that device current, on the first call for that device.
// Make that first call outside any stream capture.
constexpr size_t kNoAllocScratchFloats = 512u * 1024u;   // 2 MiB
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[kNoAllocScratchFloats];
// Per-device address of the array, shared by every context of the process: guarded by its own mutex.
static float* g_rmsnorm_bwd_scratch_addr[64] = {};
static std::mutex g_rmsnorm_bwd_scratch_mu;

int32_t t0b_rmsnorm_bwd_noalloc(t0b_ctx* ctx, uint64_t dy, uint64_t x, uint64_t weight, uint64_t dx, uint64_t dgamma,
                                uint32_t rows, uint32_t cols, float eps, int32_t async) {
    int32_t rc = precheck(ctx);   // makes ctx->device the current device
    if (rc != T0B_OK) return rc;
    if (cols == 0 || !dy || !x || !weight || !dgamma)
        return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_bwd_noalloc: null pointer or zero cols");
    const size_t need = static_cast<size_t>(rows) + static_cast<size_t>(kDgammaRowBlocks) * cols;
    if (need > kNoAllocScratchFloats)
        return set_error(ctx, T0B_ERR_INVALID,
                         "rmsnorm_bwd_noalloc: rows + %u*cols = %zu floats exceeds the built-in scratch of %zu floats "
                         "(2 MiB); use t0b_rmsnorm_bwd with caller-provided scratch",
                         kDgammaRowBlocks, need, kNoAllocScratchFloats);
    if (ctx->device < 0 || ctx->device >= 64) return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_bwd_noalloc: device index out of range");
    if (rows == 0) {
        // No rows: dgamma is a sum over nothing.  The memset is ordered on the stream like a kernel, and a synchronous
        // call waits for it like any other.
        rc = check_cuda(ctx, cudaMemsetAsync(reinterpret_cast<void*>(dgamma), 0, static_cast<size_t>(cols) * 4, ctx->stream),
                        "cudaMemsetAsync(dgamma)");
        if (rc != T0B_OK) return rc;
        return finish(ctx, async, "rmsnorm_bwd_noalloc", 0);
    }
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_rmsnorm_bwd_scratch_mu);
        scratch = g_rmsnorm_bwd_scratch_addr[ctx->device];
        if (!scratch) {
            rc = check_cuda(ctx, cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_rmsnorm_bwd_scratch),
                            "cudaGetSymbolAddress(rmsnorm scratch)");
            if (rc != T0B_OK) return rc;
            g_rmsnorm_bwd_scratch_addr[ctx->device] = scratch;
        }
    }
    // Every float the later stages read is written first by an earlier stage of this same call (inv_rms by the
    // dx stage, the used partial rows by the partial stage), so nothing left over from a previous call is seen
    // and nothing needs clearing.
    float* inv = scratch;
    float* partial = scratch + rows;
    const int threads = cols >= 2048 ? kRowThreads : (cols >= 512 ? 128 : 32);
    rmsnorm_bwd_dx_kernel<<<rows, threads, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                                                             reinterpret_cast<const float*>(weight), reinterpret_cast<float*>(dx),
                                                             inv, cols, eps);
    rc = check_cuda(ctx, cudaGetLastError(), "rmsnorm_bwd_noalloc dx launch");
    if (rc != T0B_OK) return rc;
    const uint32_t nblocks = std::min(kDgammaRowBlocks, rows);
    const uint32_t rpb = (rows + nblocks - 1) / nblocks;
    const uint32_t used = (rows + rpb - 1) / rpb;
    dim3 grid((cols + 255) / 256, used);
    rmsnorm_dgamma_partial_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(x),
                                                                 inv, partial, rows, cols, rpb);
    rc = check_cuda(ctx, cudaGetLastError(), "rmsnorm_bwd_noalloc partial launch");
    if (rc != T0B_OK) return rc;
    rmsnorm_dgamma_final_kernel<<<kDgammaFinalGrid(cols), 256, 0, ctx->stream>>>(partial, reinterpret_cast<float*>(dgamma), cols, used);
    return finish(ctx, async, "rmsnorm_bwd_noalloc", 3);
}

int32_t t0b_softmax_fwd(t0b_ctx* ctx, uint64_t x, uint64_t y, uint32_t rows, uint32_t cols, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) return T0B_OK;
    if (cols == 0 || !x || !y) return set_error(ctx, T0B_ERR_INVALID, "softmax_fwd: null pointer or zero cols");
    const int threads = cols >= 2048 ? kRowThreads : (cols >= 512 ? 128 : 32);
    const size_t bytes = static_cast<size_t>(cols) * 4;
    if (bytes <= kRowCacheMax && cols >= 2048) {
        static bool set[64] = {};
        if (!set[ctx->device & 63]) {
            rc = check_cuda(ctx, cudaFuncSetAttribute(softmax_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      static_cast<int>(kRowCacheLimit)), "cudaFuncSetAttribute(softmax)");
            if (rc != T0B_OK) return rc;
            set[ctx->device & 63] = true;
        }
        softmax_fwd_kernel<true><<<rows, threads, bytes, ctx->stream>>>(reinterpret_cast<const float*>(x), reinterpret_cast<float*>(y), cols);
    } else {
        softmax_fwd_kernel<false><<<rows, threads, 0, ctx->stream>>>(reinterpret_cast<const float*>(x), reinterpret_cast<float*>(y), cols);
    }
    return finish(ctx, async, "softmax_fwd");
}

int32_t t0b_softmax_bwd(t0b_ctx* ctx, uint64_t dy, uint64_t y, uint64_t dx, uint32_t rows, uint32_t cols, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) return T0B_OK;
    if (cols == 0 || !dy || !y || !dx) return set_error(ctx, T0B_ERR_INVALID, "softmax_bwd: null pointer or zero cols");
    const int threads = cols >= 2048 ? kRowThreads : (cols >= 512 ? 128 : 32);
    softmax_bwd_kernel<<<rows, threads, 0, ctx->stream>>>(reinterpret_cast<const float*>(dy), reinterpret_cast<const float*>(y),
                                                          reinterpret_cast<float*>(dx), cols);
    return finish(ctx, async, "softmax_bwd");
}

static int32_t softmax_ce_impl(t0b_ctx* ctx, uint64_t logits, uint64_t targets, uint64_t losses, uint64_t dlogits, uint32_t rows,
                               uint32_t cols, uint64_t ld, float scale, bool grad16, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) return T0B_OK;
    if (cols == 0 || !logits || !targets || (!losses && !dlogits) || ld < cols)
        return set_error(ctx, T0B_ERR_INVALID, "softmax_ce: null pointer, zero cols or pitch < cols");
    const int threads = cols >= 2048 ? kRowThreads : (cols >= 512 ? 128 : 32);
    const size_t bytes = static_cast<size_t>(cols) * 4;
    const float* lp = reinterpret_cast<const float*>(logits);
    const uint32_t* tp = reinterpret_cast<const uint32_t*>(targets);
    float* losp = reinterpret_cast<float*>(losses);
    void* dp = reinterpret_cast<void*>(dlogits);
    if (bytes <= kRowCacheMax && cols >= 2048) {
        static bool set[64] = {};
        if (!set[ctx->device & 63]) {
            rc = check_cuda(ctx, cudaFuncSetAttribute(softmax_ce_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      static_cast<int>(kRowCacheLimit)), "cudaFuncSetAttribute(softmax_ce)");
            if (rc == T0B_OK)
                rc = check_cuda(ctx, cudaFuncSetAttribute(softmax_ce_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                          static_cast<int>(kRowCacheLimit)), "cudaFuncSetAttribute(softmax_ce bf16)");
            if (rc != T0B_OK) return rc;
            set[ctx->device & 63] = true;
        }
        if (grad16) softmax_ce_kernel<true, true><<<rows, threads, bytes, ctx->stream>>>(lp, tp, losp, dp, cols, ld, scale);
        else softmax_ce_kernel<true, false><<<rows, threads, bytes, ctx->stream>>>(lp, tp, losp, dp, cols, ld, scale);
    } else {
        if (grad16) softmax_ce_kernel<false, true><<<rows, threads, 0, ctx->stream>>>(lp, tp, losp, dp, cols, ld, scale);
        else softmax_ce_kernel<false, false><<<rows, threads, 0, ctx->stream>>>(lp, tp, losp, dp, cols, ld, scale);
    }
    return finish(ctx, async, "softmax_ce");
}

int32_t t0b_softmax_ce(t0b_ctx* ctx, uint64_t logits, uint64_t targets, uint64_t losses, uint64_t dlogits, uint32_t rows,
                       uint32_t cols, uint64_t ld, float scale, int32_t async) {
    return softmax_ce_impl(ctx, logits, targets, losses, dlogits, rows, cols, ld, scale, false, async);
}

int32_t t0b_softmax_ce_bf16(t0b_ctx* ctx, uint64_t logits, uint64_t targets, uint64_t losses, uint64_t dlogits_bf16, uint32_t rows,
                            uint32_t cols, uint64_t ld, float scale, int32_t async) {
    return softmax_ce_impl(ctx, logits, targets, losses, dlogits_bf16, rows, cols, ld, scale, true, async);
}

int32_t t0b_silu_gate_fwd(t0b_ctx* ctx, uint64_t gate, uint64_t up, uint64_t out, size_t n, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (n == 0) return T0B_OK;
    if (!gate || !out) return set_error(ctx, T0B_ERR_INVALID, "silu_gate_fwd: null pointer");
    silu_gate_fwd_kernel<<<grid_for(ctx, n, 1024), 256, 0, ctx->stream>>>(reinterpret_cast<const float*>(gate), reinterpret_cast<const float*>(up),
                                                                         reinterpret_cast<float*>(out), n);
    return finish(ctx, async, "silu_gate_fwd");
}

int32_t t0b_silu_gate_bwd(t0b_ctx* ctx, uint64_t grad, uint64_t gate, uint64_t up, uint64_t dgate, uint64_t dup, size_t n,
                          int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (n == 0) return T0B_OK;
    if (!grad || !gate || !dgate) return set_error(ctx, T0B_ERR_INVALID, "silu_gate_bwd: null pointer");
    silu_gate_bwd_kernel<<<grid_for(ctx, n, 1024), 256, 0, ctx->stream>>>(reinterpret_cast<const float*>(grad), reinterpret_cast<const float*>(gate),
                                                                         reinterpret_cast<const float*>(up), reinterpret_cast<float*>(dgate),
                                                                         reinterpret_cast<float*>(dup), n);
    return finish(ctx, async, "silu_gate_bwd");
}

int32_t t0b_residual_add(t0b_ctx* ctx, uint64_t y, uint64_t x, size_t n, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (n == 0) return T0B_OK;
    if (!x || !y) return set_error(ctx, T0B_ERR_INVALID, "residual_add: null pointer");
    residual_add_kernel<<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>(reinterpret_cast<float*>(y), reinterpret_cast<const float*>(x), n);
    return finish(ctx, async, "residual_add");
}

int32_t t0b_adamw_step(t0b_ctx* ctx, uint64_t params, uint64_t grads, uint64_t m, uint64_t v, uint64_t params_bf16, size_t n,
                       float lr, float beta1, float beta2, float eps, float weight_decay, uint32_t t, float grad_scale,
                       int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (n == 0) return T0B_OK;
    if (!params || !grads || !m || !v || t == 0) return set_error(ctx, T0B_ERR_INVALID, "adamw_step: null pointer or t == 0");
    const float bc1 = 1.0f / (1.0f - powf(beta1, static_cast<float>(t)));
    const float bc2 = 1.0f / (1.0f - powf(beta2, static_cast<float>(t)));
    adamw_kernel<<<grid_for(ctx, n, 1024), 256, 0, ctx->stream>>>(reinterpret_cast<float*>(params), reinterpret_cast<const float*>(grads),
                                                                 reinterpret_cast<float*>(m), reinterpret_cast<float*>(v),
                                                                 reinterpret_cast<__nv_bfloat16*>(params_bf16), n, lr, beta1, beta2, eps,
                                                                 weight_decay, bc1, bc2, grad_scale);
    return finish(ctx, async, "adamw_step");
}

// ------------------------------------------------------------------------------------------------
// RMSNorm -> SiLU -> bf16 in one pass each way (the block between two Linear layers of the MLP).
// ------------------------------------------------------------------------------------------------
static bool rmsnorm_reg_path(uint64_t ptrs, uint32_t cols) {
    return (ptrs & 15) == 0 && cols % 4 == 0 && cols >= 1024 && cols <= 4u * 4u * kRowThreads;
}

int32_t t0b_rmsnorm_silu_fwd(t0b_ctx* ctx, uint64_t x, uint64_t weight, uint64_t out_bf16, uint64_t inv_rms, uint32_t rows,
                             uint32_t cols, float eps, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) return T0B_OK;
    if (cols == 0 || !x || !weight || !out_bf16) return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_silu_fwd: null pointer or zero cols");
    if (rmsnorm_reg_path(x | weight | out_bf16, cols)) {
        const uint32_t g = std::min<uint32_t>(rows, static_cast<uint32_t>(ctx->num_sms) * 4u);
        const uint32_t n4 = cols / 4;
        const float* xp = reinterpret_cast<const float*>(x);
        const float* wp = reinterpret_cast<const float*>(weight);
        void* yp = reinterpret_cast<void*>(out_bf16);
        float* ip = reinterpret_cast<float*>(inv_rms);
        if (n4 <= 1u * kRowThreads) rmsnorm_fwd_reg_kernel<1, true><<<g, kRowThreads, 0, ctx->stream>>>(xp, wp, yp, ip, rows, cols, eps);
        else if (n4 <= 2u * kRowThreads) rmsnorm_fwd_reg_kernel<2, true><<<g, kRowThreads, 0, ctx->stream>>>(xp, wp, yp, ip, rows, cols, eps);
        else rmsnorm_fwd_reg_kernel<4, true><<<g, kRowThreads, 0, ctx->stream>>>(xp, wp, yp, ip, rows, cols, eps);
        return finish(ctx, async, "rmsnorm_silu_fwd");
    }
    // Other shapes: the three kernels in sequence through a pooled f32 buffer (same values).
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    const size_t n = static_cast<size_t>(rows) * cols;
    uint64_t tmp = 0;
    rc = t0b_alloc(ctx, n * 4, &tmp);
    if (rc != T0B_OK) return rc;
    rc = t0b_rmsnorm_fwd(ctx, x, weight, tmp, inv_rms, rows, cols, eps, 1);
    if (rc == T0B_OK) rc = t0b_silu_gate_fwd(ctx, tmp, 0, tmp, n, 1);
    if (rc == T0B_OK) rc = t0b_cast_f32_to_bf16(ctx, tmp, out_bf16, n, 1);
    t0b_recycle(ctx, tmp);
    if (rc != T0B_OK) return rc;
    return finish(ctx, async, "rmsnorm_silu_fwd", 0);
}

int32_t t0b_rmsnorm_silu_bwd(t0b_ctx* ctx, uint64_t dh, uint64_t x, uint64_t weight, uint64_t dx_bf16, uint64_t dgamma,
                             uint64_t scratch, size_t scratch_bytes, uint32_t rows, uint32_t cols, float eps, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (rows == 0) {
        if (dgamma && cols) return t0b_memset0(ctx, dgamma, static_cast<size_t>(cols) * 4);
        return T0B_OK;
    }
    if (cols == 0 || !dh || !x || !weight || (!dx_bf16 && !dgamma))
        return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_silu_bwd: null pointer or zero cols");
    if (dgamma && (!scratch || scratch_bytes < t0b_rmsnorm_bwd_scratch_bytes(rows, cols)))
        return set_error(ctx, T0B_ERR_INVALID, "rmsnorm_silu_bwd: dgamma needs %zu bytes of scratch, got %zu",
                         t0b_rmsnorm_bwd_scratch_bytes(rows, cols), scratch_bytes);
    if (rmsnorm_reg_path(dh | x | weight | dx_bf16 | scratch, cols)) {
        const uint32_t g = dgamma ? rmsnorm_fused_ctas(rows) : std::min<uint32_t>(rows, static_cast<uint32_t>(ctx->num_sms) * 4u);
        const uint32_t n4 = cols / 4;
        float* partial = dgamma ? reinterpret_cast<float*>(scratch) + ((static_cast<size_t>(rows) + 3) & ~static_cast<size_t>(3)) : nullptr;
        const float* dp = reinterpret_cast<const float*>(dh);
        const float* xp = reinterpret_cast<const float*>(x);
        const float* wp = reinterpret_cast<const float*>(weight);
        void* op = reinterpret_cast<void*>(dx_bf16);
        if (n4 <= 1u * kRowThreads) rmsnorm_bwd_fused_kernel<1, true><<<g, kRowThreads, 0, ctx->stream>>>(dp, xp, wp, op, partial, rows, cols, eps);
        else if (n4 <= 2u * kRowThreads) rmsnorm_bwd_fused_kernel<2, true><<<g, kRowThreads, 0, ctx->stream>>>(dp, xp, wp, op, partial, rows, cols, eps);
        else rmsnorm_bwd_fused_kernel<4, true><<<g, kRowThreads, 0, ctx->stream>>>(dp, xp, wp, op, partial, rows, cols, eps);
        rc = check_cuda(ctx, cudaGetLastError(), "rmsnorm_silu_bwd launch");
        if (rc != T0B_OK) return rc;
        if (dgamma) {
            ++ctx->launches;
            rmsnorm_dgamma_final_kernel<<<kDgammaFinalGrid(cols), 256, 0, ctx->stream>>>(partial, reinterpret_cast<float*>(dgamma), cols, g);
        }
        return finish(ctx, async, "rmsnorm_silu_bwd");
    }
    // Other shapes: recompute the normalised row, then SiLU backward, RMSNorm backward and the cast in sequence.
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    const size_t n = static_cast<size_t>(rows) * cols;
    uint64_t r = 0, dr = 0;
    rc = t0b_alloc(ctx, n * 4, &r);
    if (rc == T0B_OK) rc = t0b_alloc(ctx, n * 4, &dr);
    if (rc == T0B_OK) rc = t0b_rmsnorm_fwd(ctx, x, weight, r, 0, rows, cols, eps, 1);
    if (rc == T0B_OK) rc = t0b_silu_gate_bwd(ctx, dh, r, 0, dr, 0, n, 1);
    if (rc == T0B_OK) rc = t0b_rmsnorm_bwd(ctx, dr, x, weight, dx_bf16 ? r : 0, dgamma, scratch, scratch_bytes, rows, cols, eps, 1);
    if (rc == T0B_OK && dx_bf16) rc = t0b_cast_f32_to_bf16(ctx, r, dx_bf16, n, 1);
    if (r) t0b_recycle(ctx, r);
    if (dr) t0b_recycle(ctx, dr);
    if (rc != T0B_OK) return rc;
    return finish(ctx, async, "rmsnorm_silu_bwd", 0);
}

}  // extern "C"
