// Small device utilities next to the GEMM path: a block-wise checksum of a buffer (to compare whole outputs across
// ranks or runs without copying them to the host) and a plain copy kernel (SM-issued 16-byte stores; pointed at a
// peer-mapped destination it measures the store rate the fused all-gather epilogue can reach over NVLink).
// No counterpart in the reference, whose tests read results through mapped VRAM
// (examples/test_gemm_correctness.rs:198-211).
#include "t0b_internal.hpp"

using namespace t0b;

namespace {

// One CTA per block of `block_bytes`: out[2*b] = wrapping sum of the block's 64-bit words, out[2*b+1] = their XOR,
// each word first mixed with its index inside the block so that swapped words change the result.
__global__ void __launch_bounds__(256) hash_blocks_kernel(const unsigned long long* __restrict__ src, size_t words,
                                                          size_t words_per_block, unsigned long long* __restrict__ out) {
    const size_t b = blockIdx.x;
    const size_t w0 = b * words_per_block;
    const size_t w1 = w0 + words_per_block < words ? w0 + words_per_block : words;
    unsigned long long s = 0, x = 0;
    for (size_t i = w0 + threadIdx.x; i < w1; i += 256) {
        const unsigned long long v = src[i];
        const unsigned long long mixed = (v ^ ((i - w0) * 0x9E3779B97F4A7C15ull)) * 0xD6E8FEB86659FD93ull;
        s += mixed;
        x ^= mixed ^ (mixed >> 29);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        x ^= __shfl_xor_sync(0xffffffffu, x, o);
    }
    __shared__ unsigned long long ss[8], sx[8];
    if ((threadIdx.x & 31) == 0) { ss[threadIdx.x >> 5] = s; sx[threadIdx.x >> 5] = x; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) { s += ss[i]; x ^= sx[i]; }   // ss[0], sx[0] are this thread's own values
        out[2 * b] = s;
        out[2 * b + 1] = x;
    }
}

__global__ void __launch_bounds__(256) copy16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t n16) {
    for (size_t i = blockIdx.x * static_cast<size_t>(256) + threadIdx.x; i < n16; i += static_cast<size_t>(gridDim.x) * 256)
        dst[i] = src[i];
}

// Rows of `width16` 16-byte pieces, with separate row pitches (in 16-byte units) on either side.
__global__ void __launch_bounds__(256) copy16_2d_kernel(uint4* __restrict__ dst, size_t dst_pitch16, const uint4* __restrict__ src,
                                                        size_t src_pitch16, size_t width16, size_t rows) {
    const size_t total = width16 * rows;
    for (size_t i = blockIdx.x * static_cast<size_t>(256) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * 256) {
        const size_t r = i / width16, c = i - r * width16;
        dst[r * dst_pitch16 + c] = src[r * src_pitch16 + c];
    }
}

}  // namespace

extern "C" {

int32_t t0b_hash_blocks(t0b_ctx* ctx, uint64_t src, size_t bytes, size_t block_bytes, uint64_t out, int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (bytes == 0) return T0B_OK;
    if (!src || !out || block_bytes == 0 || (bytes % 8) != 0 || (block_bytes % 8) != 0 || (src % 8) != 0 || (out % 8) != 0)
        return set_error(ctx, T0B_ERR_INVALID, "hash_blocks: null pointer, or sizes / pointers that are not multiples of 8 bytes");
    const size_t nblocks = (bytes + block_bytes - 1) / block_bytes;
    if (nblocks > 0x7fffffffull) return set_error(ctx, T0B_ERR_INVALID, "hash_blocks: too many blocks");
    hash_blocks_kernel<<<static_cast<unsigned>(nblocks), 256, 0, ctx->stream>>>(reinterpret_cast<const unsigned long long*>(src), bytes / 8,
                                                                                block_bytes / 8, reinterpret_cast<unsigned long long*>(out));
    return finish(ctx, async, "hash_blocks");
}

int32_t t0b_copy_d2d(t0b_ctx* ctx, uint64_t dst, size_t dst_pitch, uint64_t src, size_t src_pitch, size_t width_bytes, size_t rows,
                     int32_t async) {
    int32_t rc = precheck(ctx);
    if (rc != T0B_OK) return rc;
    if (width_bytes == 0 || rows == 0) return T0B_OK;
    if (!dst || !src || ((dst | src | dst_pitch | src_pitch | width_bytes) & 15) != 0 || dst_pitch < width_bytes || src_pitch < width_bytes)
        return set_error(ctx, T0B_ERR_INVALID, "copy_d2d: null pointer, a pitch smaller than the row, or something not a multiple of 16 bytes");
    const size_t n16 = width_bytes / 16 * rows;
    const unsigned grid = static_cast<unsigned>(std::min<size_t>((n16 + 255) / 256, static_cast<size_t>(ctx->num_sms) * 8));
    if (dst_pitch == width_bytes && src_pitch == width_bytes)
        copy16_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src), n16);
    else
        copy16_2d_kernel<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<uint4*>(dst), dst_pitch / 16, reinterpret_cast<const uint4*>(src),
                                                        src_pitch / 16, width_bytes / 16, rows);
    return finish(ctx, async, "copy_d2d");
}

}  // extern "C"
