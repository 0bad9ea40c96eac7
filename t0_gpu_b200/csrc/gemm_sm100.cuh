// bf16 x bf16 -> f32-accumulate GEMM for sm_100a: persistent, warp-specialised, TMA-fed shared-memory
// ring, tcgen05.mma with double-buffered TMEM accumulators, optional CTA pairs (cta_group::2).
//
// Replaces the reference's generated RDNA3 WMMA kernels (src/t0/gemm_gen.rs:637-1348 `generate_lds_db`,
// src/t0/tile_ir.rs:585 `lower_gemm`): same math (Y = op(A) * op(B), bf16 in, f32 accumulate), same
// split-K contract (slab s holds the partial sum of K-chunk s, src/t0/gemm_gen.rs:746-752), same edge
// behaviour as the tile_ir path (rows/cols beyond M/N are never stored, src/t0/tile_ir.rs:2462-2472;
// the K tail contributes zeros, :768-787) -- here the zero fill is TMA's out-of-bounds fill, so callers
// do not have to pad.
//
// Roles per CTA: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, then four or eight epilogue warps
// (TMEM -> registers -> shared-memory transpose tile -> TMA store or coalesced row stores): 192 threads for the
// 64-column tile, 320 otherwise.  Every wait is bounded: when a wait runs out the CTA records a status code, raises
// its abort flag, drains, frees its TMEM and returns.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

#include "ptx_sm100.cuh"

namespace t0b {

// Fused store-phase operations.  0..2 are the generator's EpilogueOp (src/t0/gemm_gen.rs:40-49); the rest
// are the tile_ir chain's single-op members (src/t0/tile_ir.rs:41-62).
enum EpilogueKind : int {
    EPI_STORE = 0,
    EPI_BIAS = 1,
    EPI_BIAS_RELU = 2,
    EPI_RELU = 3,
    EPI_SILU = 4,
    EPI_GELU_SIGMOID = 5,  // x * sigmoid(1.702 x)
    EPI_SCALE = 6,
    EPI_ABS = 7,
    EPI_NEG = 8,
    EPI_CLAMP = 9,
};

// A store-phase chain of up to four operations applied in order (the tile_ir epilogue chain,
// src/t0/tile_ir.rs:2213-2339).  EPI_BIAS_RELU never appears here: the host expands it to {EPI_BIAS, EPI_RELU}.
constexpr int kMaxEpiOps = 4;
struct EpiChain {
    int n;
    int ops[kMaxEpiOps];
    float alpha;              // EPI_SCALE factor
    float clamp_lo, clamp_hi; // EPI_CLAMP bounds
    const float* bias;        // f32[N] for EPI_BIAS
};

// Device status codes written to the context's status word.
enum DeviceStatus : int {
    DEV_OK = 0,
    DEV_TIMEOUT_EMPTY = 101,      // producer waited for a free ring slot
    DEV_TIMEOUT_FULL = 102,       // MMA issuer waited for TMA data
    DEV_TIMEOUT_TMEM_EMPTY = 103, // MMA issuer waited for the epilogue to drain an accumulator
    DEV_TIMEOUT_TMEM_FULL = 104,  // epilogue waited for an accumulator
    DEV_TIMEOUT_SELFTEST = 105,   // the bounded-wait self test (a barrier nobody arrives on)
};

constexpr int kMaxDst = 8;

struct GemmParams {
    void* c_dst[kMaxDst];   // destinations of the epilogue store: [0] local, [1..] peers of a column-sharded GEMM
    int n_dst;
    long long ldc;          // row pitch of C in elements
    EpiChain epi;           // fused store-phase operations (none when epi.n == 0)
    float* partial;         // split-K slabs (f32, slab s at partial + s * slab_stride); null when split_k == 1
    long long slab_stride;  // elements
    long long ld_partial;   // row pitch of a slab in elements
    int M, N, K;
    int tiles_m, tiles_n;   // in units of the cluster tile (128*CG x BN)
    int split_k;
    int kb_total, kb_per_split;  // K blocks of 64
    int a_mn_major, b_mn_major;  // 0: operand stored K-contiguous; 1: stored M/N-contiguous
    int out_bf16;
    int raster_along_n;     // 0: group tile rows (walk N inside a group of M tiles); 1: the transpose
    int group;              // rasterisation group width in tiles
    unsigned mn_lbo, mn_sbo, mn_kstep;  // descriptor byte offsets for M/N-contiguous operands
    int* status;
    unsigned long long wait_limit_ns;
    int tma_store;          // 1: the epilogue writes C with TMA stores through the third tensor map
    unsigned wait_hint_ns;  // suspend-time hint of the epilogue warps' wait for an accumulator
#ifdef T0B_TRACE
    unsigned long long* trace;   // timeline build only: [CTA][16] stamps of this launch (null = no stamps)
#endif
    int cluster_sk;         // > 1: split-K inside a thread-block cluster of that many CTAs (one per K range): the partial
                            // tiles stay in shared memory and are summed over distributed shared memory; 0 = slabs
};

constexpr int kBmCta = 128;   // accumulator rows per MMA per CTA (TMEM lanes)
constexpr int kBk = 64;       // K block: 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kASubTileBytes = kBmCta * kBk * 2;   // one 128-row A tile of a stage

// BN: MMA N (tile width).  CG: CTAs sharing one MMA (1, or 2 = cta_group::2 pair).  MT: 128-row A tiles per CTA.
//   MT = 1: the two TMEM accumulator slots double-buffer consecutive tiles (epilogue of tile i overlaps the main
//           loop of tile i+1); tile = (128*CG) x BN.
//   MT = 2: both slots belong to the same tile, which is (256*CG) x BN: every B tile is used by two MMAs, so the
//           shared-memory fill traffic per FLOP drops by a quarter; each slot has its own epilogue warp group and
//           the slots drain in parallel.
template <int BN, int CG, int MT, int ND = 0>
struct GemmTraits {
    static_assert(BN == 64 || BN == 128 || BN == 256, "BN");
    static_assert(CG == 1 || CG == 2, "CG");
    static_assert(MT == 1 || MT == 2, "MT");
    static_assert(ND == 0 || (ND == 1 && MT == 2), "the N-direction double tile uses both accumulator slots");
    // ND == 1: the two slots hold two N-adjacent tiles that share one A tile (tile = (128*CG) x (2*BN)); consecutive
    // MMAs then take A from the tensor core's collector, which removes a quarter of the operand reads from shared
    // memory compared with two M-adjacent tiles sharing B.
    static constexpr int kATiles = ND ? 1 : MT;
    static constexpr int kBTiles = ND ? 2 : 1;
    static constexpr int kBnCta = BN / CG;               // B rows this CTA loads
    static_assert(kBnCta % 64 == 0, "each CTA's B slice must be whole 64-column swizzle blocks");
    static constexpr int kATileBytes = kATiles * kASubTileBytes;
    static constexpr int kBSubTileBytes = kBnCta * kBk * 2;
    static constexpr int kBTileBytes = kBTiles * kBSubTileBytes;
    static constexpr int kStageBytes = kATileBytes + kBTileBytes;
    static constexpr int kCtrlBytes = 1024;   // keeps the transpose tiles behind it 1024-byte aligned (TMA swizzle)
    // Single-accumulator tiles of at least 128 columns are drained by two groups of four warps, each taking half of the
    // columns: the epilogue of the last tile of a CTA is exposed, and it is the store sequence of one warp per lane
    // quarter, not the memory system, that bounds it.
    static constexpr int kEpiSplit = (MT == 1 && BN >= 128) ? 2 : 1;
    static constexpr int kEpiWarps = 4 * MT * kEpiSplit;
    static constexpr int kEpiStagingBytes = kEpiWarps * 4096;   // one 32x32 f32 transpose tile per epilogue warp
    static constexpr int kBudget = 227 * 1024 - 1024 - kCtrlBytes - kEpiStagingBytes;
    static constexpr int kStagesRaw = kBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
    static constexpr int kTmemCols = 2 * BN;             // two accumulator slots
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + kCtrlBytes + kEpiStagingBytes;
    static constexpr int kThreads = 64 + 32 * kEpiWarps;
    static constexpr int kBm = kBmCta * CG * kATiles;    // rows of the cluster tile
    static constexpr int kTileN = BN * kBTiles;          // columns of the cluster tile
};

struct WorkItem {
    int m0, n0, split, kb_begin, kb_end;
};

__device__ __forceinline__ WorkItem decode_work(const GemmParams& p, int w, int bm, int bn) {
    const int num_tiles = p.tiles_m * p.tiles_n;
    // Cluster split-K: the CTAs of a cluster (consecutive work items) are the K ranges of one tile.
    const int split = p.cluster_sk > 1 ? w % p.cluster_sk : w / num_tiles;
    const int tile = p.cluster_sk > 1 ? w / p.cluster_sk : w - split * num_tiles;
    int major_cnt = p.raster_along_n ? p.tiles_n : p.tiles_m;   // dimension that is grouped
    int minor_cnt = p.raster_along_n ? p.tiles_m : p.tiles_n;
    const int per_group = p.group * minor_cnt;
    const int g = tile / per_group;
    const int first = g * p.group;
    const int gsz = min(major_cnt - first, p.group);
    const int in_group = tile - g * per_group;
    const int major = first + in_group % gsz;
    const int minor = in_group / gsz;
    WorkItem wi;
    wi.m0 = (p.raster_along_n ? minor : major) * bm;
    wi.n0 = (p.raster_along_n ? major : minor) * bn;
    wi.split = split;
    wi.kb_begin = split * p.kb_per_split;
    wi.kb_end = min(p.kb_total, wi.kb_begin + p.kb_per_split);
    return wi;
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;   // descriptor version for sm_100
    d |= 2ull << 61;   // SWIZZLE_128B
    return d;
}

// Timeline build (-DT0B_TRACE, libt0b200_trace.so): one thread per role stamps %globaltimer (slots 12 / 13 of a
// non-split-K launch: clock64, so that cycles / nanoseconds gives the SM clock of the main loop) into
// trace[blockIdx.x][slot].  The regular build compiles the stamps away.
//   0 kernel entry            1 set-up done (barriers, TMEM)   2 dependency wait returned     3 first K block issued (producer)
//   4 first operands arrived  5 last MMA issued                6 accumulator complete (epilogue warp 0)
//   7 last chunk staged       8 this warp's stores complete    9 teardown barrier passed      10 all loads issued
//  12 cluster split-K: closing barrier passed (else clock64 at 4)    13 cluster split-K: partials visible (else clock64 at 5)
//  14 TMEM freed
#ifdef T0B_TRACE
#define T0B_STAMP(slot) do { if (p.trace) p.trace[blockIdx.x * 16 + (slot)] = ptx::globaltimer_ns(); } while (0)
#define T0B_STAMP_CLOCK(slot) do { if (p.trace) p.trace[blockIdx.x * 16 + (slot)] = static_cast<unsigned long long>(clock64()); } while (0)
#else
#define T0B_STAMP(slot) do { } while (0)
#define T0B_STAMP_CLOCK(slot) do { } while (0)
#endif

struct WaitCtl {
    volatile int* abort;
    int* status;
    unsigned long long limit_ns;
};

// Bounded mbarrier wait.  Returns false when the limit ran out or another thread of the CTA aborted.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const WaitCtl& ctl, int code) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0) {
            if (*ctl.abort) return false;
            if (ptx::globaltimer_ns() - t0 > ctl.limit_ns) {
                *ctl.abort = 1;
                *reinterpret_cast<volatile int*>(ctl.status) = code;
                return false;
            }
        }
    }
}

// The same wait for a whole warp: lane 0 polls (with a suspend-time hint, so the thread sleeps in hardware between
// polls instead of spinning beside the MMA issuer for a whole main loop), the result is broadcast.
__device__ __forceinline__ bool bounded_wait_warp(uint32_t bar, uint32_t parity, const WaitCtl& ctl, int code, int lane,
                                                  uint32_t hint_ns) {
    int ok = 1;
    if (lane == 0) {
        ok = 0;
        if (ptx::mbar_try_wait_hint(bar, parity, hint_ns)) ok = 1;
        else {
            const uint64_t t0 = ptx::globaltimer_ns();
            while (true) {
                if (ptx::mbar_try_wait_hint(bar, parity, hint_ns)) { ok = 1; break; }
                if (*ctl.abort) break;
                if (ptx::globaltimer_ns() - t0 > ctl.limit_ns) {
                    *ctl.abort = 1;
                    *reinterpret_cast<volatile int*>(ctl.status) = code;
                    break;
                }
            }
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__device__ __forceinline__ bool chain_has_bias(const EpiChain& e) {
    bool b = false;
    for (int i = 0; i < e.n; ++i) b = b || (e.ops[i] == EPI_BIAS);
    return b && e.bias != nullptr;
}

__device__ __forceinline__ float apply_chain(float v, const EpiChain& e, float bias) {
    for (int i = 0; i < e.n; ++i) {
        switch (e.ops[i]) {
            case EPI_BIAS: v = v + bias; break;
            case EPI_RELU: v = fmaxf(v, 0.0f); break;
            case EPI_SILU: v = v / (1.0f + __expf(-v)); break;
            case EPI_GELU_SIGMOID: v = v / (1.0f + __expf(-1.702f * v)); break;
            case EPI_SCALE: v = v * e.alpha; break;
            case EPI_ABS: v = fabsf(v); break;
            case EPI_NEG: v = -v; break;
            case EPI_CLAMP: v = fminf(fmaxf(v, e.clamp_lo), e.clamp_hi); break;
            default: break;
        }
    }
    return v;
}

// Store one thread's 32 consecutive output columns of one row.
__device__ __forceinline__ void store_chunk_f32(float* base, long long ld, int row, int col0, int ncols_valid,
                                                const float (&v)[32], bool vec_ok) {
    float* dst = base + static_cast<long long>(row) * ld + col0;
    if (vec_ok && ncols_valid >= 32) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < ncols_valid) dst[j] = v[j];
    }
}

__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* base, long long ld, int row, int col0, int ncols_valid,
                                                 const float (&v)[32], bool vec_ok) {
    __nv_bfloat16* dst = base + static_cast<long long>(row) * ld + col0;
    if (vec_ok && ncols_valid >= 32) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint4 q;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
            q.x = *reinterpret_cast<uint32_t*>(&h0);
            q.y = *reinterpret_cast<uint32_t*>(&h1);
            q.z = *reinterpret_cast<uint32_t*>(&h2);
            q.w = *reinterpret_cast<uint32_t*>(&h3);
            reinterpret_cast<uint4*>(dst)[j] = q;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < ncols_valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}


// Coalesced stores of one warp's 32x32 chunk (lane i holds row i) through a 4 KiB shared-memory transpose tile.
// 16-byte pieces are XOR-swizzled by row so both the row-wise writes and the line-wise reads are conflict-free.
// Each global store instruction then writes whole 128-byte (f32) or 64-byte (bf16) row segments.
__device__ __forceinline__ void stage_chunk_f32(uint32_t stage, int lane, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t addr = stage + lane * 128 + ((j ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                     "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                     : "memory");
    }
}
__device__ __forceinline__ void flush_chunk_f32(uint32_t stage, int lane, float* base, long long ld, int row0, int col0,
                                                int M, int N) {
    const int c = lane & 7;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int r = t * 4 + (lane >> 3);
        const uint32_t addr = stage + r * 128 + ((c ^ (r & 7)) << 4);
        float4 q;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(q.x), "=f"(q.y), "=f"(q.z), "=f"(q.w) : "r"(addr));
        if (row0 + r < M && col0 + c * 4 < N)   // N % 4 == 0 on this path, so a piece is all in or all out
            *reinterpret_cast<float4*>(base + static_cast<long long>(row0 + r) * ld + col0 + c * 4) = q;
    }
}
// TMA-store path: every 32x32 chunk goes out through two 2 KiB half tiles (rows of 64 bytes, 64-byte TMA swizzle:
// 16-byte piece c of row r sits at piece c ^ ((r >> 1) & 3)), so that one half is being read by its TMA store while
// the warp fills the other.  f32: a half holds 16 of the chunk's columns; bf16: a half holds one whole chunk.
__device__ __forceinline__ void stage_half_f32_sw64(uint32_t half_tile, int lane, const float* v) {
    const uint32_t row = half_tile + lane * 64;
    const int x = (lane >> 1) & 3;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(row + ((j ^ x) << 4)), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                     "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                     : "memory");
}
__device__ __forceinline__ void stage_chunk_bf16_sw64(uint32_t half_tile, int lane, const float (&v)[32]) {
    const uint32_t row = half_tile + lane * 64;
    const int x = (lane >> 1) & 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row + ((j ^ x) << 4)), "r"(*reinterpret_cast<uint32_t*>(&h0)),
                     "r"(*reinterpret_cast<uint32_t*>(&h1)), "r"(*reinterpret_cast<uint32_t*>(&h2)),
                     "r"(*reinterpret_cast<uint32_t*>(&h3))
                     : "memory");
    }
}
// bf16 output: two 32-column chunks share one tile (32 rows x 64 bf16 = 128-byte rows), so the flush writes
// whole 128-byte lines, local or remote.
__device__ __forceinline__ void stage_half_bf16(uint32_t stage, int lane, int half, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
        const uint32_t addr = stage + lane * 128 + (((half * 4 + j) ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(*reinterpret_cast<uint32_t*>(&h0)),
                     "r"(*reinterpret_cast<uint32_t*>(&h1)), "r"(*reinterpret_cast<uint32_t*>(&h2)),
                     "r"(*reinterpret_cast<uint32_t*>(&h3))
                     : "memory");
    }
}
__device__ __forceinline__ void flush_pair_bf16(uint32_t stage, int lane, __nv_bfloat16* base, long long ld, int row0,
                                                int col0, int M, int N) {
    const int c = lane & 7;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int r = t * 4 + (lane >> 3);
        const uint32_t addr = stage + r * 128 + ((c ^ (r & 7)) << 4);
        uint4 q;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(addr));
        if (row0 + r < M && col0 + c * 8 < N)   // N % 8 == 0 on this path
            *reinterpret_cast<uint4*>(base + static_cast<long long>(row0 + r) * ld + col0 + c * 8) = q;
    }
}

template <int BN, int CG, int MT, int ND = 0>
__global__ void __launch_bounds__(GemmTraits<BN, CG, MT, ND>::kThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    using T = GemmTraits<BN, CG, MT, ND>;
    constexpr int S = T::kStages;
    constexpr int BM = T::kBm;
    constexpr int BNT = T::kTileN;
    constexpr int kMmaM = kBmCta * CG;    // rows of one MMA (128 or 256)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
    uint8_t* smem_gen = smem_raw + (smem_base - raw_addr);

    const uint32_t ctrl = smem_base + S * T::kStageBytes;
    auto full_bar = [&](int s) { return ctrl + 8u * s; };
    auto empty_bar = [&](int s) { return ctrl + 8u * (S + s); };
    auto tfull_bar = [&](int a) { return ctrl + 8u * (2 * S + a); };
    auto tempty_bar = [&](int a) { return ctrl + 8u * (2 * S + 2 + a); };
    const uint32_t slot_off = 8u * (2 * S + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + S * T::kStageBytes + slot_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + S * T::kStageBytes + slot_off + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0) T0B_STAMP(0);
    const uint32_t cta_rank = (CG == 2) ? ptx::cluster_ctarank() : 0u;
    const bool is_leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(tfull_bar(a), 1);
            ptx::mbar_init(tempty_bar(a), 4 * CG * T::kEpiSplit);   // one arrival per epilogue warp of the slot, from every CTA of the group
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tmap(&tmap_a);
        ptx::prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<CG>(ctrl + slot_off, T::kTmemCols);
        ptx::tmem_relinquish<CG>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (CG == 2) {
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Cluster split-K (single-CTA tiles only): the CTAs of the cluster are the K ranges of one tile.
    const bool csk = (CG == 1 && MT == 1) && p.cluster_sk > 1;
    const WaitCtl ctl{abort_flag, p.status, p.wait_limit_ns};
    const int num_work = p.tiles_m * p.tiles_n * p.split_k;
    const int cluster_id = blockIdx.x / CG;
    const int num_clusters = gridDim.x / CG;
    // The first work item is decoded here, before the dependency wait: the parameter reads and the divisions of the
    // decode (half a microsecond on a cold SM, measured with globaltimer stamps) then overlap the previous kernel's
    // tail.  The empty asm pins the values in front of the wait.
    const WorkItem first_wi = decode_work(p, cluster_id < num_work ? cluster_id : 0, BM, BNT);
    asm volatile("" ::"r"(first_wi.m0), "r"(first_wi.n0), "r"(first_wi.kb_begin), "r"(first_wi.kb_end), "r"(first_wi.split));
    if (threadIdx.x == 0) T0B_STAMP(1);
    // Programmatic dependent launch: everything above (barriers, TMEM, descriptor prefetch) may run while the previous
    // kernel of the stream drains; nothing below may touch global memory before that kernel has completed.
    ptx::grid_dependency_wait();
    if (threadIdx.x == 0) T0B_STAMP(2);
    ptx::grid_launch_dependents();   // the next GEMM's CTAs may take over SMs as this grid's CTAs exit

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int w = cluster_id; w < num_work && ok; w += num_clusters) {
                const WorkItem wi = (w == cluster_id) ? first_wi : decode_work(p, w, BM, BNT);
                const int m0_cta = wi.m0 + static_cast<int>(cta_rank) * kBmCta;
                const int n0_cta = wi.n0 + static_cast<int>(cta_rank) * T::kBnCta;
                for (int kb = wi.kb_begin; kb < wi.kb_end; ++kb) {
                    if (!bounded_wait(empty_bar(s), ph ^ 1u, ctl, DEV_TIMEOUT_EMPTY)) { ok = false; break; }
                    if (is_leader) ptx::mbar_arrive_expect_tx(full_bar(s), CG * T::kStageBytes);
                    const uint32_t a_dst = smem_base + s * T::kStageBytes;
                    const uint32_t b_dst = a_dst + T::kATileBytes;
                    const int k0 = kb * kBk;
                    // The pair's barrier lives in CTA 0; a single CTA uses its own.
                    const uint32_t bar = (CG == 2) ? ptx::mapa(full_bar(s), 0) : full_bar(s);
                    auto load = [&](uint32_t dst, const CUtensorMap* m, int c0, int c1) {
                        if constexpr (CG == 1) ptx::tma_load_2d(dst, m, bar, c0, c1);
                        else ptx::tma_load_2d_pair(dst, m, bar, c0, c1);
                    };
#pragma unroll
                    for (int mt = 0; mt < T::kATiles; ++mt) {
                        const int m_sub = m0_cta + mt * kMmaM;
                        const uint32_t dst = a_dst + mt * kASubTileBytes;
                        if (!p.a_mn_major) {
                            load(dst, &tmap_a, k0, m_sub);
                        } else {
                            load(dst, &tmap_a, m_sub, k0);
                            load(dst + 8192, &tmap_a, m_sub + 64, k0);
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < T::kBTiles; ++nt) {
                        const int n_sub = n0_cta + nt * BN;
                        const uint32_t dst = b_dst + nt * T::kBSubTileBytes;
                        if (!p.b_mn_major) {
                            load(dst, &tmap_b, k0, n_sub);
                        } else {
#pragma unroll
                            for (int j = 0; j < T::kBnCta / 64; ++j) load(dst + j * 8192, &tmap_b, n_sub + j * 64, k0);
                        }
                    }
                    if (w == cluster_id && kb == wi.kb_begin) T0B_STAMP(3);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
            T0B_STAMP(10);
            // Tail: every slot must have been released, so no MMA-completion arrival can target this
            // CTA's shared memory after it exits.
            for (int i = 0; i < S && ok; ++i) {
                if (!bounded_wait(empty_bar(s), ph ^ 1u, ctl, DEV_TIMEOUT_EMPTY)) ok = false;
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && is_leader) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(p.a_mn_major) << 15) |
                                   (static_cast<uint32_t>(p.b_mn_major) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                   (static_cast<uint32_t>(kMmaM >> 4) << 24);
            const uint32_t a_lbo = p.a_mn_major ? p.mn_lbo : 16u, a_sbo = p.a_mn_major ? p.mn_sbo : 1024u;
            const uint32_t b_lbo = p.b_mn_major ? p.mn_lbo : 16u, b_sbo = p.b_mn_major ? p.mn_sbo : 1024u;
            const uint32_t a_kstep = p.a_mn_major ? p.mn_kstep : 32u;
            const uint32_t b_kstep = p.b_mn_major ? p.mn_kstep : 32u;
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;                       // MT == 1: the slot of this tile
            uint32_t slot_ph[2] = {0u, 0u};    // phase of each accumulator slot
            bool ok = true;
            for (int w = cluster_id; w < num_work && ok; w += num_clusters) {
                const WorkItem wi = (w == cluster_id) ? first_wi : decode_work(p, w, BM, BNT);
                if constexpr (MT == 1) {
                    if (!bounded_wait(tempty_bar(acc), slot_ph[acc] ^ 1u, ctl, DEV_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
                    ptx::tc_fence_after();
                }
                for (int kb = wi.kb_begin; kb < wi.kb_end; ++kb) {
                    if (!bounded_wait(full_bar(s), ph, ctl, DEV_TIMEOUT_FULL)) { ok = false; break; }
                    if (w == cluster_id && kb == wi.kb_begin) {
                        T0B_STAMP(4);
                        if (!csk) T0B_STAMP_CLOCK(12);
                    }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = smem_base + s * T::kStageBytes;
                    const uint32_t b_addr = a_addr + T::kATileBytes;
#pragma unroll
                    for (int k = 0; k < kBk / kUmmaK; ++k) {
                        const uint32_t acc_flag = (kb > wi.kb_begin || k > 0) ? 1u : 0u;
                        if constexpr (ND == 1) {
                            // One A slice, two B slices: the second MMA takes A from the collector.
                            const uint64_t adesc = make_smem_desc(a_addr + k * a_kstep, a_lbo, a_sbo);
#pragma unroll
                            for (int nt = 0; nt < 2; ++nt) {
                                if (kb == wi.kb_begin && k == 0) {
                                    if (!bounded_wait(tempty_bar(nt), slot_ph[nt] ^ 1u, ctl, DEV_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
                                    ptx::tc_fence_after();
                                }
                                const uint64_t bdesc = make_smem_desc(b_addr + nt * T::kBSubTileBytes + k * b_kstep, b_lbo, b_sbo);
                                if (nt == 0) ptx::mma_f16<CG, 1>(tmem_base + 0u, adesc, bdesc, idesc, acc_flag);
                                else ptx::mma_f16<CG, 2>(tmem_base + static_cast<uint32_t>(BN), adesc, bdesc, idesc, acc_flag);
                            }
                        } else {
                            const uint64_t bdesc = make_smem_desc(b_addr + k * b_kstep, b_lbo, b_sbo);
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                const int slot = (MT == 1) ? acc : mt;
                                if (MT == 2 && kb == wi.kb_begin && k == 0) {
                                    // First write into this slot for the tile: its previous contents must be drained.
                                    if (!bounded_wait(tempty_bar(slot), slot_ph[slot] ^ 1u, ctl, DEV_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
                                    ptx::tc_fence_after();
                                }
                                const uint64_t adesc = make_smem_desc(a_addr + mt * kASubTileBytes + k * a_kstep, a_lbo, a_sbo);
                                ptx::mma_f16<CG>(tmem_base + static_cast<uint32_t>(slot * BN), adesc, bdesc, idesc, acc_flag);
                            }
                        }
                        if (!ok) break;
                    }
                    if (!ok) break;
                    if constexpr (CG == 1) ptx::mma_commit(empty_bar(s));
                    else ptx::mma_commit_pair(empty_bar(s), 0x3);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                T0B_STAMP(5);
                if (!csk) T0B_STAMP_CLOCK(13);
                if constexpr (MT == 1) {
                    if constexpr (CG == 1) ptx::mma_commit(tfull_bar(acc));
                    else ptx::mma_commit_pair(tfull_bar(acc), 0x3);
                    slot_ph[acc] ^= 1u;
                    acc ^= 1;
                } else {
#pragma unroll
                    for (int slot = 0; slot < 2; ++slot) {
                        if constexpr (CG == 1) ptx::mma_commit(tfull_bar(slot));
                        else ptx::mma_commit_pair(tfull_bar(slot), 0x3);
                        slot_ph[slot] ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue: one group of 4 warps per slot owner
        const int q = warp & 3;              // TMEM lane quarter this warp may read
        const int group = (warp - 2) >> 2;   // MT == 2: group g drains slot g of every tile; else group g takes column half g
        int slot = (MT == 2) ? group : 0;
        constexpr int kChunks = BN / 32 / T::kEpiSplit;          // 32-column chunks per warp and tile
        const int c_begin = (T::kEpiSplit == 2) ? group * kChunks : 0;
        uint32_t slot_phase = 0;
        const bool to_slab = p.split_k > 1 && !csk;
        const long long ld_out = to_slab ? p.ld_partial : p.ldc;
        bool vec_ok;
        if (to_slab || !p.out_bf16) {
            vec_ok = (ld_out % 4 == 0);
            if (to_slab) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.partial) & 15) == 0) && (p.slab_stride % 4 == 0);
            else for (int d = 0; d < p.n_dst; ++d) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.c_dst[d]) & 15) == 0);
        } else {
            vec_ok = (ld_out % 8 == 0);
            for (int d = 0; d < p.n_dst; ++d) vec_ok = vec_ok && ((reinterpret_cast<uintptr_t>(p.c_dst[d]) & 15) == 0);
        }
        const bool has_epi = !to_slab && p.epi.n > 0;
        const bool need_bias = has_epi && chain_has_bias(p.epi);
        // The transposing path needs whole 16-byte pieces inside [0, N): N % 4 (f32) or N % 8 (bf16).
        const bool out16 = !to_slab && p.out_bf16;
        const bool tma_out = p.tma_store != 0;   // implies one destination, no slabs, TMA-addressable C
        const bool staged = tma_out || (vec_ok && (p.N % (out16 ? 8 : 4) == 0));
        if (tma_out && lane == 0) ptx::prefetch_tmap(&tmap_c);
        const uint32_t stage = ctrl + T::kCtrlBytes + static_cast<uint32_t>(warp - 2) * 4096u;
        for (int w = cluster_id; w < num_work; w += num_clusters) {
            const WorkItem wi = (w == cluster_id) ? first_wi : decode_work(p, w, BM, BNT);
            if (!bounded_wait_warp(tfull_bar(slot), slot_phase, ctl, DEV_TIMEOUT_TMEM_FULL, lane, p.wait_hint_ns)) break;
            if (warp == 2 && lane == 0) T0B_STAMP(6);
            ptx::tc_fence_after();
            const int row0 = wi.m0 + ((MT == 2 && ND == 0) ? group * kMmaM : 0) + static_cast<int>(cta_rank) * kBmCta + q * 32;
            const int n_base = wi.n0 + (ND == 1 ? group * BN : 0);
            const int row = row0 + lane;
            const uint32_t t_row = tmem_base + static_cast<uint32_t>(slot * BN) + (static_cast<uint32_t>(q * 32) << 16);
            // The TMEM read of chunk c+1 is in flight while chunk c is transposed and stored.
            uint32_t nxt[32];
            ptx::tmem_ld_32x32(t_row + c_begin * 32, nxt);
#pragma unroll 2
            for (int c = c_begin; c < c_begin + kChunks; ++c) {
                uint32_t raw[32];
                ptx::tmem_ld_wait_regs(nxt);
#pragma unroll
                for (int j = 0; j < 32; ++j) raw[j] = nxt[j];
                if (c + 1 < c_begin + kChunks) ptx::tmem_ld_32x32(t_row + (c + 1) * 32, nxt);
                if (c == c_begin + kChunks - 1) {
                    // All of this warp's reads of the accumulator are done: hand it back to the MMA issuer.
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CG == 1) ptx::mbar_arrive(tempty_bar(slot));
                        else ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(slot), 0));
                    }
                }
                const int col0 = n_base + c * 32;
                const int ncols = p.N - col0;
                if (csk) {
                    // The partial tile goes to shared memory (the operand ring is idle: this CTA has one work item and
                    // its last MMA has completed), row-major [128][BN] f32 with the 16-byte pieces of every 128-byte
                    // segment XOR-swizzled by row, for the cluster-wide sum after the barrier below.
                    const int rl = q * 32 + lane;
                    const uint32_t seg = smem_base + static_cast<uint32_t>(rl * BN * 4 + c * 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(seg + ((j ^ (rl & 7)) << 4)), "r"(raw[4 * j]),
                                     "r"(raw[4 * j + 1]), "r"(raw[4 * j + 2]), "r"(raw[4 * j + 3])
                                     : "memory");
                } else if (tma_out && out16) {
                    if (row0 < p.M && ncols > 0) {   // warp-uniform
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                        if (has_epi) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float b = 0.0f;
                                if (need_bias && j < ncols) b = __ldg(p.epi.bias + col0 + j);
                                v[j] = apply_chain(v[j], p.epi, b);
                            }
                        }
                        const uint32_t half_tile = stage + static_cast<uint32_t>(c & 1) * 2048u;
                        if (lane == 0) ptx::bulk_wait_group_read<1>();   // the store that last used this half has read it
                        __syncwarp();
                        stage_chunk_bf16_sw64(half_tile, lane, v);
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            ptx::tma_store_2d(&tmap_c, half_tile, col0, row0);
                            ptx::bulk_commit_group();
                        }
                    }
                } else if (staged && out16) {
                    const int half = c & 1;
                    if (half == 0) __syncwarp();   // the previous pair's reads of the staging tile are done
                    if (row0 < p.M && ncols > 0) {   // warp-uniform
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                        if (has_epi) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float b = 0.0f;
                                if (need_bias && j < ncols) b = __ldg(p.epi.bias + col0 + j);
                                v[j] = apply_chain(v[j], p.epi, b);
                            }
                        }
                        stage_half_bf16(stage, lane, half, v);
                    }
                    if (half == 1) {
                        __syncwarp();
                        const int cbase = col0 - 32;
                        if (row0 < p.M && cbase < p.N) {
                            for (int d = 0; d < p.n_dst; ++d)
                                flush_pair_bf16(stage, lane, static_cast<__nv_bfloat16*>(p.c_dst[d]), ld_out, row0, cbase, p.M, p.N);
                        }
                    }
                } else if (staged) {
                    if (row0 < p.M && ncols > 0) {   // warp-uniform
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                        if (has_epi) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float b = 0.0f;
                                if (need_bias && j < ncols) b = __ldg(p.epi.bias + col0 + j);
                                v[j] = apply_chain(v[j], p.epi, b);
                            }
                        }
                        if (tma_out) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const uint32_t half_tile = stage + static_cast<uint32_t>(h) * 2048u;
                                if (lane == 0) ptx::bulk_wait_group_read<1>();   // the store that last used this half has read it
                                __syncwarp();
                                stage_half_f32_sw64(half_tile, lane, v + 16 * h);
                                ptx::fence_proxy_async_smem();
                                __syncwarp();
                                if (lane == 0 && col0 + 16 * h < p.N) {
                                    ptx::tma_store_2d(&tmap_c, half_tile, col0 + 16 * h, row0);
                                    ptx::bulk_commit_group();
                                }
                            }
                            continue;
                        }
                        __syncwarp();   // the previous chunk's reads of the staging tile are done
                        stage_chunk_f32(stage, lane, v);
                        __syncwarp();
                        if (to_slab) {
                            flush_chunk_f32(stage, lane, p.partial + static_cast<long long>(wi.split) * p.slab_stride, ld_out,
                                            row0, col0, p.M, p.N);
                        } else {
                            for (int d = 0; d < p.n_dst; ++d)
                                flush_chunk_f32(stage, lane, static_cast<float*>(p.c_dst[d]), ld_out, row0, col0, p.M, p.N);
                        }
                    }
                } else if (row < p.M && ncols > 0) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                    if (has_epi) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            float b = 0.0f;
                            if (need_bias && j < ncols) b = __ldg(p.epi.bias + col0 + j);
                            v[j] = apply_chain(v[j], p.epi, b);
                        }
                    }
                    if (to_slab) {
                        store_chunk_f32(p.partial + static_cast<long long>(wi.split) * p.slab_stride, ld_out, row, col0,
                                        ncols, v, vec_ok);
                    } else if (p.out_bf16) {
                        for (int d = 0; d < p.n_dst; ++d)
                            store_chunk_bf16(static_cast<__nv_bfloat16*>(p.c_dst[d]), ld_out, row, col0, ncols, v, vec_ok);
                    } else {
                        for (int d = 0; d < p.n_dst; ++d)
                            store_chunk_f32(static_cast<float*>(p.c_dst[d]), ld_out, row, col0, ncols, v, vec_ok);
                    }
                }
            }
            if constexpr (MT == 1) {
                slot ^= 1;
                if (slot == 0) slot_phase ^= 1u;
            } else {
                slot_phase ^= 1u;
            }
        }
        if (warp == 2 && lane == 0) T0B_STAMP(7);
        if (tma_out && lane == 0) ptx::bulk_wait_group<0>();   // every TMA store of this warp has completed
        if (warp == 2 && lane == 0) T0B_STAMP(8);
    }

    if (csk) {
        // Every CTA of the cluster has its partial tile in shared memory after this barrier (release / acquire at
        // cluster scope).  CTA r then sums rows [r, r+1) * 128 / sk of the tile over the sk partials IN K-RANGE ORDER,
        // starting from +0.0 -- the arithmetic of splitk_reduce_kernel and of the reference's host-side slab sum
        // (examples/test_gemm_correctness.rs:203-207) -- and writes them to C.  No slab ever reaches global memory.
        // This phase takes 3.9 us of a 13.5 us kernel (128x128 tile, four K ranges), and every alternative measured
        // slower: sixteen loads in flight per thread instead of four (+1.3 us: the distributed-shared-memory path
        // congests), pushing the rows to their owners with st.shared::cluster (+2.2 us), and exchanging the partials
        // through slabs in L2 with the same cluster barrier between the stores and the loads (+3.9 us).
        ptx::cluster_arrive();
        ptx::cluster_wait();
        if (threadIdx.x == 64) T0B_STAMP(13);
        if (warp >= 2 && !*abort_flag) {
            const int sk = p.cluster_sk;
            const WorkItem& wi = first_wi;   // a cluster split-K CTA has exactly one work item (CG == 1: cluster_id == blockIdx.x)
            const int rows_per = kBmCta / sk;
            constexpr int kPiecesPerRow = BN / 4;
            const int total = rows_per * kPiecesPerRow;
            const bool need_bias = chain_has_bias(p.epi);
            const bool vec_c = (p.N % 4 == 0) && (p.ldc % (p.out_bf16 ? 2 : 4) == 0) &&
                               ((reinterpret_cast<uintptr_t>(p.c_dst[0]) & 15) == 0) && (!p.out_bf16 || p.ldc % 4 == 0);
            for (int i = static_cast<int>(threadIdx.x) - 64; i < total; i += T::kEpiWarps * 32) {
                const int rl = wi.split * rows_per + i / kPiecesPerRow;
                const int pc = i % kPiecesPerRow;
                const uint32_t off = smem_base + static_cast<uint32_t>(rl * BN * 4 + (pc >> 3) * 128 + (((pc & 7) ^ (rl & 7)) << 4));
                float4 part[8];
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx)
                    if (sidx < sk) part[sidx] = ptx::ld_shared_cluster_v4(ptx::mapa(off, static_cast<uint32_t>(sidx)));
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx)
                    if (sidx < sk) {
                        acc[0] = acc[0] + part[sidx].x; acc[1] = acc[1] + part[sidx].y;
                        acc[2] = acc[2] + part[sidx].z; acc[3] = acc[3] + part[sidx].w;
                    }
                const int row = wi.m0 + rl, col = wi.n0 + pc * 4;
                if (row >= p.M || col >= p.N) continue;
                if (p.epi.n > 0) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        acc[e] = apply_chain(acc[e], p.epi, (need_bias && col + e < p.N) ? __ldg(p.epi.bias + col + e) : 0.0f);
                }
                if (p.out_bf16) {
                    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c_dst[0]) + static_cast<long long>(row) * p.ldc + col;
                    if (vec_c) {
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]);
                        uint2 qv;
                        qv.x = *reinterpret_cast<uint32_t*>(&h0);
                        qv.y = *reinterpret_cast<uint32_t*>(&h1);
                        *reinterpret_cast<uint2*>(dst) = qv;
                    } else {
                        for (int e = 0; e < 4 && col + e < p.N; ++e) dst[e] = __float2bfloat16_rn(acc[e]);
                    }
                } else {
                    float* dst = static_cast<float*>(p.c_dst[0]) + static_cast<long long>(row) * p.ldc + col;
                    if (vec_c) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                    else for (int e = 0; e < 4 && col + e < p.N; ++e) dst[e] = acc[e];
                }
            }
        }
        // Nobody leaves while a peer may still read its shared memory.
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }

    // ---------------------------------------------------------------------- teardown (normal and abort paths)
    if (csk && threadIdx.x == 64) T0B_STAMP(12);
    ptx::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) T0B_STAMP(9);
    if (*abort_flag) {
        // Give this CTA's own TMA copies in flight time to land before the shared memory is released.
        const uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    if constexpr (CG == 2) {
        // The peer may still read this CTA's tiles / signal its barriers until both are done.
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<CG>(tmem_base, T::kTmemCols);
        if (lane == 0) T0B_STAMP(14);
    }
}

// The kernels below are not templates: they are compiled in the dispatch file only, not once per tile variant.
#ifndef T0B_VARIANT
// ---------------------------------------------------------------------------------------------------------
// Deterministic split-K reduce: out[i] = epilogue(sum over s = 0..sk-1, in that order, of slab_s[i]),
// starting from +0.0 -- the order of the reference's host-side slab sum
// (examples/test_gemm_correctness.rs:203-207).  One thread per 4 consecutive columns.
// ---------------------------------------------------------------------------------------------------------
struct ReduceParams {
    const float* partial;
    long long slab_stride, ld_partial;
    void* c;
    long long ldc;
    EpiChain epi;
    int M, N, sk, out_bf16;
};

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const ReduceParams p) {
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();   // launched behind the GEMM that writes the slabs (programmatic serialization)
    const int n4 = (p.N + 3) / 4;
    const long long total = static_cast<long long>(p.M) * n4;
    const bool vec_in = (p.ld_partial % 4 == 0) && (p.slab_stride % 4 == 0) &&
                        ((reinterpret_cast<uintptr_t>(p.partial) & 15) == 0);
    const bool vec_out = p.out_bf16 ? false
                                    : ((p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0));
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / n4);
        const int col = static_cast<int>(i - static_cast<long long>(row) * n4) * 4;
        const int nv = min(4, p.N - col);
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* src = p.partial + static_cast<long long>(row) * p.ld_partial + col;
        for (int s = 0; s < p.sk; ++s) {
            const float* ps = src + static_cast<long long>(s) * p.slab_stride;
            if (vec_in && nv == 4) {
                const float4 v = *reinterpret_cast<const float4*>(ps);
                acc[0] = acc[0] + v.x; acc[1] = acc[1] + v.y; acc[2] = acc[2] + v.z; acc[3] = acc[3] + v.w;
            } else {
                for (int j = 0; j < nv; ++j) acc[j] = acc[j] + ps[j];
            }
        }
        const bool need_bias = chain_has_bias(p.epi);
        for (int j = 0; j < nv; ++j) acc[j] = apply_chain(acc[j], p.epi, need_bias ? p.epi.bias[col + j] : 0.0f);
        if (p.out_bf16) {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.c) + static_cast<long long>(row) * p.ldc + col;
            for (int j = 0; j < nv; ++j) dst[j] = __float2bfloat16_rn(acc[j]);
        } else {
            float* dst = static_cast<float*>(p.c) + static_cast<long long>(row) * p.ldc + col;
            if (vec_out && nv == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            else for (int j = 0; j < nv; ++j) dst[j] = acc[j];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Plain CUDA-core GEMM for operands TMA cannot address (row pitch not a multiple of 16 bytes, or a base
// pointer that is not 16-byte aligned).  Correctness path only: 64x64 tile, 16x16 threads, 4x4 per thread.
// ---------------------------------------------------------------------------------------------------------
struct SimtParams {
    const __nv_bfloat16 *a, *b;
    void* c;
    EpiChain epi;
    long long lda, ldb, ldc;
    int M, N, K, trans_a, trans_b, out_bf16;
    int k_begin, k_end;
};

__global__ void __launch_bounds__(256) gemm_bf16_simt_kernel(const SimtParams p) {
    __shared__ float As[16][64 + 1];
    __shared__ float Bs[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = p.k_begin; k0 < p.k_end; k0 += 16) {
        for (int i = threadIdx.x; i < 16 * 64; i += 256) {
            const int kk = i & 15, mm = i >> 4;
            const int gk = k0 + kk, gm = m0 + mm, gn = n0 + mm;
            float av = 0.0f, bv = 0.0f;
            if (gk < p.k_end && gm < p.M)
                av = __bfloat162float(p.trans_a ? p.a[static_cast<long long>(gk) * p.lda + gm]
                                                : p.a[static_cast<long long>(gm) * p.lda + gk]);
            if (gk < p.k_end && gn < p.N)
                bv = __bfloat162float(p.trans_b ? p.b[static_cast<long long>(gn) * p.ldb + gk]
                                                : p.b[static_cast<long long>(gk) * p.ldb + gn]);
            As[kk][mm] = av;
            Bs[kk][mm] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    const bool need_bias = chain_has_bias(p.epi);
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) {
            const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
            if (gm < p.M && gn < p.N) {
                const float v = apply_chain(acc[i][j], p.epi, need_bias ? p.epi.bias[gn] : 0.0f);
                if (p.out_bf16) static_cast<__nv_bfloat16*>(p.c)[static_cast<long long>(gm) * p.ldc + gn] = __float2bfloat16_rn(v);
                else static_cast<float*>(p.c)[static_cast<long long>(gm) * p.ldc + gn] = v;
            }
        }
}

// Bounded-wait self test: one thread waits on a barrier nobody arrives on; the wait must run out, record
// DEV_TIMEOUT_SELFTEST and return, leaving the context usable.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        ptx::fence_mbar_init();
        const WaitCtl ctl{&abort_flag, status, limit_ns};
        bounded_wait(ptx::smem_u32(&bar), 0, ctl, DEV_TIMEOUT_SELFTEST);
    }
}

#endif  // T0B_VARIANT
}  // namespace t0b
