// Internal declarations shared by the translation units of libt0b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/t0b200.h"

struct t0b_ctx {
    int device = 0;
    int num_sms = 148;
    bool pdl = true;            // launch GEMMs with programmatic stream serialization (T0B_PDL=0 turns it off)
    int raster_group = 0;       // > 0: rasterisation group width for every GEMM (T0B_RASTER_GROUP, for measurements); 0 = chosen per shape
    bool cluster_splitk = true; // split-K of single-CTA tiles runs as thread-block clusters (T0B_CLUSTER_SPLITK=0: slabs + reduce kernel)
    std::string force_config;   // T0_FORCE_CONFIG=<preset name>: the tile every GEMM without an explicit config runs
    bool dump_config = false;   // T0_DUMP_CONFIG=1: print the config and the kernel variant of each new GEMM shape to stderr
    std::map<std::string, int> dumped;
    unsigned wait_hint_ns = 20000;   // T0B_WAIT_HINT_NS: how long an epilogue warp may sleep in hardware per poll of its accumulator barrier
    // Timeline build: where the stamps of the next GEMM launches go (t0b_trace_set); unused in the regular build.
    uint64_t trace_buf = 0;
    uint32_t trace_slots = 0, trace_next = 0;
    int sm_limit = 0;           // > 0: the persistent GEMM kernels occupy at most this many SMs
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    std::recursive_mutex mu;
    std::string last_error;
    bool poisoned = false;
    // Device status word: pinned host memory mapped into the device, so a kernel can report that one of its
    // bounded waits ran out without any copy.
    int* status_host = nullptr;
    int* status_dev = nullptr;
    unsigned long long wait_limit_ns = 2000000000ull;
    int last_status = 0;        // the code most recently taken from the status word (kept for t0b_device_status)
    // Buffer pool keyed by 4 KiB-rounded size.
    std::multimap<size_t, void*> pool_free;
    std::unordered_map<void*, size_t> live;
    uint64_t pool_cached = 0, pool_hits = 0, pool_misses = 0;
    // Grow-only split-K workspace.
    void* ws = nullptr;
    size_t ws_bytes = 0;
    // bf16 copies of f32 weight buffers, by caller-chosen tensor id (GpuRuntime::bf16_cache, src/ignis/gpu_context.rs:392-432).
    struct Bf16Entry { uint64_t ptr; size_t n; };
    std::unordered_map<uint64_t, Bf16Entry> bf16_cache;
    uint64_t bf16_conversions = 0, bf16_hits = 0;
    // Tensor-map cache.
    struct TmapKey {
        uint64_t ptr, d0, d1, ld;
        uint32_t b0, b1, elem;
        bool operator==(const TmapKey& o) const {
            return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && ld == o.ld && b0 == o.b0 && b1 == o.b1 && elem == o.elem;
        }
    };
    struct TmapHash {
        size_t operator()(const TmapKey& k) const {
            uint64_t h = k.ptr * 0x9E3779B97F4A7C15ull;
            h ^= (k.d0 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
            h ^= (k.d1 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
            h ^= (k.ld + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
            h ^= ((static_cast<uint64_t>(k.b0) << 32 | k.b1) + (h << 6) + (h >> 2));
            h ^= (k.elem + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
            return static_cast<size_t>(h);
        }
    };
    std::unordered_map<TmapKey, CUtensorMap, TmapHash> tmaps;
    // Graph capture.
    bool capturing = false;
    std::unordered_map<uint64_t, cudaGraphExec_t> graphs;
    uint64_t next_graph = 1;
    uint64_t launches = 0;
    std::string autotune_dir;   // empty: the disk cache is not consulted
    // Copy streams of the host-buffer GEMM (created on first use).
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    bool d2h_pending = false;   // an asynchronous read-back was queued since the last t0b_sync
    cudaStream_t p2p_stream = nullptr;   // device-to-device / peer copies that run beside the compute stream
    bool p2p_pending = false;
};

namespace t0b {

int32_t set_error(t0b_ctx* ctx, int32_t code, const char* fmt, ...);
int32_t check_cuda(t0b_ctx* ctx, cudaError_t e, const char* what);
// Status-word code of a kernel that met an index outside its table (the access is skipped); 101..105 are the GEMM's
// bounded waits.
constexpr int kDevBadIndex = 110;
int32_t precheck(t0b_ctx* ctx);                 // null / poisoned checks, sets the device
// Launch-error check (+ sync and status-word check when !async). `count` kernels are added to the launch counter.
int32_t finish(t0b_ctx* ctx, int32_t async, const char* what, int count = 1);
// Read the status word; a non-zero code is moved to ctx->last_status and the word is cleared, so one failed kernel is
// reported by one call and does not fail the calls after it.
int take_device_status(t0b_ctx* ctx);

// Host-side GemmConfig logic (t0b_gemm_gen.cpp).
void default_b200_config(uint32_t m, uint32_t k, uint32_t n, int num_sms, t0b_gemm_config* out);

// Measured configs (t0b_gemm_gen.cpp): results of t0b_tune in this process, then the table shipped with the library.
bool tuned_lookup(uint32_t m, uint32_t n, uint32_t k, int trans_a, int trans_b, int out_bf16, t0b_gemm_config* out, int* source);
void tuned_remember(uint32_t m, uint32_t n, uint32_t k, int trans_a, int trans_b, int out_bf16, const t0b_gemm_config& cfg);
void tuned_forget(uint32_t m, uint32_t n, uint32_t k);

struct PlanInput {
    uint32_t m, n, k;
    int trans_a, trans_b;
    uint64_t lda, ldb;
    uint64_t a_ptr, b_ptr;
    int num_sms;
};
void resolve_plan(const t0b_gemm_config* cfg, const PlanInput& in, t0b_gemm_plan* out);
// tile_ir front end (t0b_tile_ir.cpp): spec validation and the offsets of the epilogue arguments in its kernarg blob.
bool tile_spec_valid(const t0b_tile_gemm* spec);
size_t tile_kernarg_layout(const t0b_tile_gemm* spec, size_t* bias_off, size_t* scale_off, size_t* clamp_off);

}  // namespace t0b
