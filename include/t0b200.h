/*
 * t0b200.h -- C ABI of libt0b200.so: the B200 (sm_100a) implementation of T0-GPU's bf16 GEMM hot path.
 *
 * This is the boundary a binding of the reference's Rust crate (an `extern "C"` -sys module), a C++
 * program or Python ctypes links against.  Plain pointers and sizes only.  Device pointers are passed
 * as uint64_t, like the reference's `GpuBuffer::gpu_addr()` (src/kfd/mod.rs:947-1055).
 *
 * Conventions
 *   - every function that can fail returns int32_t: 0 = ok, negative = T0B_ERR_*; the message is
 *     available from t0b_last_error(ctx) (the reference returns Result<_, String>).
 *   - after any CUDA error the context is "poisoned" and refuses further launches, as the reference's
 *     GpuRuntime does after a queue timeout (src/ignis/gpu_context.rs:149-157, 270-272, 284-287).
 *   - there is no CPU fallback: without a CUDA device t0b_ctx_create fails.
 *   - a context is thread-safe; all launches of a context go to one CUDA stream.
 */
#ifndef T0B200_H
#define T0B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define T0B_API __attribute__((visibility("default")))
#else
#define T0B_API
#endif

typedef struct t0b_ctx t0b_ctx;

enum {
    T0B_OK = 0,
    T0B_ERR_INVALID = -1,    /* bad argument (dims, alignment, null pointer, undersized buffer) */
    T0B_ERR_CUDA = -2,       /* a CUDA runtime/driver call failed; context is poisoned */
    T0B_ERR_POISONED = -3,   /* context refused the call because an earlier error poisoned it */
    T0B_ERR_DEVICE = -4,     /* a kernel reported a device status code (bounded wait ran out) */
    T0B_ERR_NOMEM = -5,
    T0B_ERR_UNSUPPORTED = -6
};

/* ------------------------------------------------------------------------------------------------
 * GemmConfig and the generator front-end (host only, no context needed).
 * Mirrors `struct GemmConfig` and friends, src/t0/gemm_gen.rs:23-84.
 * ---------------------------------------------------------------------------------------------- */

enum { T0B_TRANSPOSE_NT = 0, T0B_TRANSPOSE_NN = 1 };                       /* GemmTranspose, gemm_gen.rs:23-33 */
enum { T0B_EPI_STORE_F32 = 0, T0B_EPI_BIAS_ADD = 1, T0B_EPI_BIAS_ADD_RELU = 2, /* EpilogueOp, gemm_gen.rs:40-49 */
       T0B_EPI_RELU = 3, T0B_EPI_SILU = 4, T0B_EPI_GELU_SIGMOID = 5,           /* tile_ir EpilogueOp members,   */
       T0B_EPI_SCALE = 6, T0B_EPI_ABS = 7, T0B_EPI_NEG = 8, T0B_EPI_CLAMP = 9 }; /* src/t0/tile_ir.rs:41-62     */
enum { T0B_OUT_F32 = 0, T0B_OUT_BF16 = 1 };

typedef struct t0b_gemm_config {
    uint32_t tile_m, tile_n, tile_k;
    uint32_t wg_size;
    uint32_t use_lds, double_buffer;
    uint32_t split_k;        /* 0 = None (the reference's Option<u32>) */
    uint32_t lds_pad, n_col_passes;   /* lds_pad: RDNA3 LDS row padding in the reference; here, when non-zero, the
                                         rasterisation group width in tiles (a pure speed knob like the original: the
                                         tuner sets it, results never depend on it) */
    uint32_t swap_grid, wgp_mode;
    uint32_t transpose;      /* T0B_TRANSPOSE_* (a name tag in the reference; the data layout is given per call) */
    uint32_t epilogue;       /* T0B_EPI_* */
} t0b_gemm_config;

/* What a GemmConfig resolves to on B200: the kernel variant that will actually run. */
typedef struct t0b_gemm_plan {
    uint32_t bm, bn, bk;       /* cluster tile: bm = 128 * cta_group * m_tiles */
    uint32_t cta_group;        /* 1, or 2 = CTA pair sharing one tcgen05.mma (tile_m >= 256) */
    uint32_t m_tiles;          /* 128-row A tiles per CTA: 1, or 2 (tile_m >= 512: both TMEM accumulators serve one tile) */
    uint32_t n_tiles;          /* N-adjacent accumulators per tile: 1, or 2 (tile_n >= 512: bn = 2 x 256, A shared) */
    uint32_t stages;
    uint32_t split_k;          /* effective split (>= 1); may be lower than asked when K has too few 64-blocks */
    uint32_t kb_per_split;     /* 64-wide K blocks per split */
    uint32_t use_tma;          /* 0 = operands not TMA-addressable, CUDA-core kernel is used */
    uint32_t grid;             /* CTAs launched */
    uint32_t smem_bytes;
} t0b_gemm_plan;

/* GemmConfig presets by name ("16x64_k16", "32x64_direct", "32x64_k16", "32x64_k32", "32x128_k16", "64x64_k16",
 * "64x64_k32", "128x64_k16", "64x128_k16", "128x64_k32", "128x128_k16", "64x64_k64", "128x128_2pass",
 * "64x128_2pass"): gemm_gen.rs:86-145.  B200-native presets: "b200_128x64", "b200_128x128", "b200_128x256",
 * "b200_256x128", "b200_256x256", "b200_512x256", "b200_256x512". */
T0B_API int32_t t0b_config_preset(const char* name, t0b_gemm_config* out);
/* GemmConfig::name(), gemm_gen.rs:207-227 (the kernel-cache / autotune key). Returns the length written. */
T0B_API int32_t t0b_config_name(const t0b_gemm_config* cfg, char* buf, size_t cap);
/* sweep_configs(), gemm_gen.rs:231-243; standard_configs(), :382-399. Return the count (<= cap written). */
T0B_API int32_t t0b_sweep_configs(t0b_gemm_config* out, int32_t cap);
T0B_API int32_t t0b_standard_configs(t0b_gemm_config* out, int32_t cap);
/* Derived getters, gemm_gen.rs:147-205. */
T0B_API uint32_t t0b_config_lds_total(const t0b_gemm_config* cfg);
T0B_API uint32_t t0b_config_estimated_vgprs(const t0b_gemm_config* cfg);
T0B_API int32_t t0b_config_is_feasible(const t0b_gemm_config* cfg);

/* auto_select(m, k, n): gemm_gen.rs:320-322.  NOTE the argument order (M, K, N).  Answers, in this order, from
 * (2) what t0b_tune measured for the shape in this process, (1) the table measured on B200 that is compiled into the
 * library (csrc/t0b_tuned_table.inc: the benchmark shapes and their backward shapes), (0) a cost model whose
 * constants were measured on B200 -- the reference's predict_best over its tune cache
 * (src/t0/cost_model.rs:593-601, 788-1078).  The call carries no layout: the NT / f32 row is preferred.
 * t0b_auto_select_source is the same lookup for one layout and output type and returns which source answered
 * (2, 1 or 0; negative on error); config-less t0b_gemm calls use exactly this lookup. */
T0B_API int32_t t0b_auto_select(uint32_t m, uint32_t k, uint32_t n, t0b_gemm_config* out);
T0B_API int32_t t0b_auto_select_source(uint32_t m, uint32_t k, uint32_t n, int32_t trans_a, int32_t trans_b,
                                       int32_t out_dtype, t0b_gemm_config* out);
/* auto_select_legacy(m, k, n): gemm_gen.rs:331-379, the 7-branch heuristic kept for A/B comparison. */
T0B_API int32_t t0b_auto_select_legacy(uint32_t m, uint32_t k, uint32_t n, t0b_gemm_config* out);
/* auto_select_backward_{data,weight}(m, n_orig, k_orig): gemm_gen.rs:482-486, 517-521. */
T0B_API int32_t t0b_auto_select_backward_data(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0b_gemm_config* out);
T0B_API int32_t t0b_auto_select_backward_weight(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0b_gemm_config* out);

/* compute_grid / compute_grid_split_k / compute_grid_auto: gemm_gen.rs:286-309, 402-409.  Grid x is in
 * THREADS (tiles * wg_size) exactly as the reference returns it. split_k must be a power of two. */
T0B_API int32_t t0b_compute_grid(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy);
T0B_API int32_t t0b_compute_grid_split_k(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t split_k,
                                         uint32_t* gx, uint32_t* gy);
T0B_API int32_t t0b_compute_grid_auto(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy);
/* compute_grid_backward_{data,weight}: gemm_gen.rs:505-508, 539-542. */
T0B_API int32_t t0b_compute_grid_backward_data(const t0b_gemm_config* cfg, uint32_t m, uint32_t k_orig, uint32_t* gx,
                                               uint32_t* gy);
T0B_API int32_t t0b_compute_grid_backward_weight(const t0b_gemm_config* cfg, uint32_t n_orig, uint32_t k_orig,
                                                 uint32_t* gx, uint32_t* gy);

/* build_kernargs(x, wt, y, k, n, m, cfg) -> 40 bytes: gemm_gen.rs:414-430.  NOTE the order (k, n, m).
 * Layout [X:u64, WT:u64, Y:u64, K:u32, N:u32, 0:u32, y_split_stride:u32], little endian. */
T0B_API int32_t t0b_build_kernargs(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                   const t0b_gemm_config* cfg, uint8_t out[40]);
/* build_kernargs_with_bias -> 48 bytes (bias pointer at 40..48): gemm_gen.rs:438-456. */
T0B_API int32_t t0b_build_kernargs_with_bias(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                             const t0b_gemm_config* cfg, uint64_t bias, uint8_t out[48]);
/* tile_ir::build_kernargs_m -> 44 bytes (M at 40..44, y_split_stride always 0): src/t0/tile_ir.rs:3173-3190. */
T0B_API int32_t t0b_build_kernargs_m(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                     uint8_t out[44]);
/* build_kernargs_backward_{data,weight}: gemm_gen.rs:495-502, 529-536. */
T0B_API int32_t t0b_build_kernargs_backward_data(uint64_t dy, uint64_t w, uint64_t dx, uint32_t m, uint32_t n_orig,
                                                 uint32_t k_orig, const t0b_gemm_config* cfg, uint8_t out[40]);
T0B_API int32_t t0b_build_kernargs_backward_weight(uint64_t dy_t, uint64_t x_t, uint64_t dw, uint32_t m,
                                                   uint32_t n_orig, uint32_t k_orig, const t0b_gemm_config* cfg,
                                                   uint8_t out[40]);

/* Resolve a GemmConfig for a problem to the B200 kernel variant (no launch, no device needed when
 * num_sms > 0 is given; pass 0 to use 148). */
T0B_API int32_t t0b_resolve_plan(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t k, int32_t trans_a,
                                 int32_t trans_b, uint64_t lda, uint64_t ldb, int32_t num_sms, t0b_gemm_plan* out);

/* ------------------------------------------------------------------------------------------------
 * Runtime: context, device memory, copies.  Replaces GpuRuntime (src/ignis/gpu_context.rs:30-106, 113-483)
 * and the KFD objects under it (KfdDevice / GpuBuffer / AqlQueue / DispatchPool, src/kfd/mod.rs).
 * ---------------------------------------------------------------------------------------------- */

/* GpuRuntime::new(), gpu_context.rs:113.  Fails (T0B_ERR_CUDA) when no CUDA device is usable.
 * Environment read here (the reference's knobs are T0_DUMP_ASM / T0_OPT_LEVEL / T0_VALIDATE_KA, src/t0/compile.rs:1149,
 * src/t0/opt_passes.rs:30, src/ignis/gpu_context.rs:277; these are their counterparts for a library without a compiler):
 *   T0_FORCE_CONFIG=<preset>  every GEMM called without a config runs this preset (t0b_config_preset names);
 *   T0_DUMP_CONFIG=1          one stderr line per new GEMM shape: config name, who chose it (caller, forced, tuned in
 *                             this process, shipped table, cost model) and the kernel variant it resolves to;
 *   T0B_PDL=0                 launches without programmatic stream serialization;
 *   T0B_CLUSTER_SPLITK=0      split-K always through slabs and the reduce kernel;
 *   T0B_RASTER_GROUP=<n>      rasterisation group width for every GEMM (a measurement knob);
 *   T0B_WAIT_HINT_NS=<ns>     suspend-time hint of the epilogue warps' accumulator wait (default 20000; 0 = busy polling,
 *                             measured 1.4 % slower at 8192^3 and no faster on the launch-bound shapes).
 * Kernarg blobs are always validated (the reference does so under T0_VALIDATE_KA). */
T0B_API int32_t t0b_ctx_create(int32_t device, t0b_ctx** out);
T0B_API void t0b_ctx_destroy(t0b_ctx* ctx);
/* Launch on a caller-owned cudaStream_t (e.g. the current stream of a host framework); NULL restores the
 * context's own stream.  The reference has a single AQL queue per runtime (src/kfd/mod.rs:1141). */
T0B_API int32_t t0b_ctx_set_stream(t0b_ctx* ctx, void* cuda_stream);
T0B_API void* t0b_ctx_stream(t0b_ctx* ctx);
T0B_API const char* t0b_last_error(t0b_ctx* ctx);
/* GpuRuntime::is_poisoned(), gpu_context.rs:149-157. */
T0B_API int32_t t0b_is_poisoned(t0b_ctx* ctx);
T0B_API int32_t t0b_num_sms(t0b_ctx* ctx);
/* The GEMM kernels are persistent: by default one CTA (or CTA pair) per SM, which leaves a concurrently running
 * kernel on another stream -- a collective of the data-parallel step -- no SM until the GEMM ends.  With a limit the
 * GEMMs occupy at most `sms` SMs (0 = all).  No reference counterpart (single GPU, one queue). */
T0B_API int32_t t0b_set_sm_limit(t0b_ctx* ctx, int32_t sms);
/* Device status word written by kernels whose bounded waits ran out (101..105) or that met an index outside its
 * table (110); 0 = none.  The first synchronous call (or t0b_sync) that finds it set returns T0B_ERR_DEVICE once and
 * takes the code out of the word, so later calls are not failed by it; the context is not poisoned.  This function
 * returns the code still in the word, else the code most recently taken, and keeps returning it until a call with
 * a non-zero `clear` forgets both.  Asynchronous calls never look at the word: after a batch of them call t0b_sync.
 * Takes the place of the reference's wait_read_ptr timeout (src/kfd/mod.rs:1607-1642). */
T0B_API int32_t t0b_device_status(t0b_ctx* ctx, int32_t clear);
/* Limit of every in-kernel wait, in nanoseconds (default 2e9). */
T0B_API int32_t t0b_set_wait_limit_ns(t0b_ctx* ctx, uint64_t ns);

/* GpuRuntime::alloc / alloc_zero / recycle, gpu_context.rs:437-457; BufferPool keyed by 4 KiB-rounded size, :48.
 * t0b_alloc takes from the pool first; t0b_recycle returns a buffer to the pool; t0b_free releases it. */
T0B_API int32_t t0b_alloc(t0b_ctx* ctx, size_t bytes, uint64_t* dptr);
T0B_API int32_t t0b_alloc_zero(t0b_ctx* ctx, size_t bytes, uint64_t* dptr);
T0B_API int32_t t0b_recycle(t0b_ctx* ctx, uint64_t dptr);
T0B_API int32_t t0b_free(t0b_ctx* ctx, uint64_t dptr);
/* BufferPool::cached_bytes, gpu_context.rs:76-78, plus hit/miss counters. */
T0B_API int32_t t0b_pool_stats(t0b_ctx* ctx, uint64_t* cached_bytes, uint64_t* hits, uint64_t* misses);
/* GpuBuffer::write / read / zero, src/kfd/mod.rs:962-1040: explicit copies (the reference maps VRAM into the
 * host).  Synchronous with respect to the host. */
T0B_API int32_t t0b_memcpy_h2d(t0b_ctx* ctx, uint64_t dst, const void* src, size_t bytes);
T0B_API int32_t t0b_memcpy_d2h(t0b_ctx* ctx, void* dst, uint64_t src, size_t bytes);
T0B_API int32_t t0b_memset0(t0b_ctx* ctx, uint64_t dst, size_t bytes);
/* Strided device -> host copy of `height` rows of `width_bytes` (a column block of a row-major matrix). */
T0B_API int32_t t0b_memcpy2d_d2h(t0b_ctx* ctx, void* dst, size_t dst_pitch, uint64_t src, size_t src_pitch,
                                 size_t width_bytes, size_t height);
/* Asynchronous forms for pinned host memory, the batched counterpart of the reference's write / dispatch_async /
 * wait_idle pattern (src/ignis/gpu_context.rs:297-332).  t0b_memcpy_h2d_async: the copy runs on the context's upload
 * stream behind the work queued so far; launches made after the call wait for it.  t0b_memcpy2d_d2h_async: the
 * read-back runs on the context's download stream behind the work queued so far, launches made after the call do NOT
 * wait for it (a strip of C travels to the host while the next strip is multiplied); t0b_sync waits for it.  The host
 * buffers must stay valid until t0b_sync returns. */
T0B_API int32_t t0b_memcpy_h2d_async(t0b_ctx* ctx, uint64_t dst, const void* src, size_t bytes);
T0B_API int32_t t0b_memcpy2d_d2h_async(t0b_ctx* ctx, void* dst, size_t dst_pitch, uint64_t src, size_t src_pitch,
                                       size_t width_bytes, size_t height);
/* GpuRuntime::synchronize / wait_idle, gpu_context.rs:297-332.  Also checks the device status word. */
T0B_API int32_t t0b_sync(t0b_ctx* ctx);

/* Share a device allocation between the one-process-per-GPU ranks of a node: export gives a 64-byte handle
 * (cudaIpcMemHandle_t) for a buffer obtained from t0b_alloc; open maps a peer's buffer into this process and
 * enables peer access over NVLink; close unmaps it.  No counterpart in the reference (single GPU). */
T0B_API int32_t t0b_ipc_export(t0b_ctx* ctx, uint64_t dptr, uint8_t handle[64]);
T0B_API int32_t t0b_ipc_open(t0b_ctx* ctx, const uint8_t handle[64], uint64_t* dptr);
T0B_API int32_t t0b_ipc_close(t0b_ctx* ctx, uint64_t dptr);

/* ------------------------------------------------------------------------------------------------
 * GEMM dispatch
 * ---------------------------------------------------------------------------------------------- */

/* C[M,N] = epilogue(op(A) * op(B)), bf16 inputs, f32 accumulate.
 *   trans_a = 0: A is [M,K] with row pitch lda;  1: A is [K,M] with row pitch lda.
 *   trans_b = 0: B is [K,N] with row pitch ldb ("NN");  1: B is [N,K] with row pitch ldb ("NT", the
 *   reference kernels' only native layout, src/t0/gemm_gen.rs:25).
 *   cfg may be NULL (auto_select).  out_dtype: T0B_OUT_F32 / T0B_OUT_BF16 (RNE).  epilogue: T0B_EPI_*; bias f32[N].
 *   Split-K (cfg->split_k > 1) on a single-CTA tile (tile_m <= 128) with 2, 4 or 8 K ranges runs as thread-block
 *   clusters: the CTAs of a cluster take the K ranges of one tile, keep the partial tiles in shared memory and sum
 *   them over distributed shared memory in K-range order, in the same launch; no workspace is used.  Otherwise
 *   (CTA-pair tiles, 16 ranges) it needs split_k*M*N*4 bytes of workspace -- pass one, or 0 to let the context keep a
 *   grow-only workspace -- and a second kernel sums the slabs in slab order.  Either way the sum runs over the K
 *   ranges in order from +0.0, so both paths, t0b_gemm_slabs + t0b_splitk_reduce and the reference's host-side slab
 *   sum (examples/test_gemm_correctness.rs:203-207) give the same bits, run after run.
 *   async = 0 waits for completion (GpuRuntime::dispatch, gpu_context.rs:264); 1 only enqueues (dispatch_async, :332).
 * Entry point behind ops::bf16_matmul::dispatch_gemm_forward / gemm_backward_data / gemm_backward_weight
 * (src/ignis/ops/bf16_matmul.rs:162-308), which stage transposes on the host instead. */
T0B_API int32_t t0b_gemm(t0b_ctx* ctx, const t0b_gemm_config* cfg, int32_t trans_a, int32_t trans_b, uint64_t a,
                         uint64_t b, uint64_t c, uint32_t m, uint32_t n, uint32_t k, uint64_t lda, uint64_t ldb,
                         uint64_t ldc, int32_t out_dtype, int32_t epilogue, uint64_t bias, float alpha,
                         uint64_t workspace, size_t workspace_bytes, int32_t async);
/* The same GEMM with a chain of up to four store-phase operations applied in order, the tile_ir epilogue chain
 * (`TileGemm::add_epilogue`, src/t0/tile_ir.rs:41-62, lowered at :2213-2339): BiasAdd (bias f32[N]), Scale (scale),
 * ReLU, SiLU, GELU (the reference's x*sigmoid(1.702x) form), Abs, Neg, Clamp (clamp_min, clamp_max). */
T0B_API int32_t t0b_gemm_chain(t0b_ctx* ctx, const t0b_gemm_config* cfg, int32_t trans_a, int32_t trans_b, uint64_t a,
                               uint64_t b, uint64_t c, uint32_t m, uint32_t n, uint32_t k, uint64_t lda, uint64_t ldb,
                               uint64_t ldc, int32_t out_dtype, const int32_t* ops, int32_t n_ops, uint64_t bias,
                               float scale, float clamp_min, float clamp_max, uint64_t workspace, size_t workspace_bytes,
                               int32_t async);
T0B_API size_t t0b_gemm_workspace_bytes(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t k);

/* The same product with A, B and C in HOST memory (what a caller of the reference sees through its host-mapped
 * buffers).  A is cut into blocks of `chunk_rows` output rows (0 = automatic, about eight blocks) and B into up to
 * eight column panels; step s uploads A block s and B panel s, and every strip of C whose operands are then resident
 * is multiplied at once and copied back while the next step uploads, on three streams.  With pinned host memory both
 * copy directions and the math overlap; pageable memory works but serialises.  Every element is accumulated over the
 * whole K in one pass (an automatically chosen config never splits K here), so the result has the same bits for every
 * blocking and equals t0b_gemm without split-K.  Device staging buffers come from the context's pool.  Synchronous:
 * returns when C is complete in host memory.  (The reference's counterpart is the write / dispatch / read sequence on
 * mapped VRAM, examples/test_gemm_correctness.rs:136-211.) */
T0B_API int32_t t0b_gemm_host(t0b_ctx* ctx, const t0b_gemm_config* cfg, int32_t trans_a, int32_t trans_b, const void* a,
                              const void* b, void* c, uint32_t m, uint32_t n, uint32_t k, uint64_t lda, uint64_t ldb,
                              uint64_t ldc, int32_t out_dtype, uint32_t chunk_rows);

/* Block-wise checksum of a device buffer: for every block of `block_bytes` (the last may be short) two 64-bit values
 * are written to out[2*b], out[2*b+1] (a position-mixed wrapping sum and XOR of the block's 64-bit words).  Equal
 * buffers give equal checksums; it lets ranks compare whole outputs (2 GiB per rank in the sharded GEMM) by exchanging
 * a few KiB.  bytes, block_bytes, src and out must be multiples of 8.  No counterpart in the reference, whose tests
 * read the full result through mapped VRAM (examples/test_gemm_correctness.rs:198-211). */
T0B_API int32_t t0b_hash_blocks(t0b_ctx* ctx, uint64_t src, size_t bytes, size_t block_bytes, uint64_t out, int32_t async);
/* Copy `rows` rows of `width_bytes` between device buffers with SM-issued 16-byte loads and stores (all sizes, pitches
 * and pointers multiples of 16).  Either side may be a peer-mapped pointer (t0b_ipc_open): with a peer destination it
 * measures the NVLink store rate that bounds the fused all-gather of t0b_gemm_multi_dst.  No reference counterpart. */
T0B_API int32_t t0b_copy_d2d(t0b_ctx* ctx, uint64_t dst, size_t dst_pitch, uint64_t src, size_t src_pitch,
                             size_t width_bytes, size_t rows, int32_t async);
/* The same copy on a copy engine, asynchronously: it runs on a side stream of the context behind the work queued so
 * far, launches made after the call do not wait for it, and t0b_sync waits for it.  With a peer-mapped destination it
 * moves a finished panel of C to a peer over NVLink while the next panel is multiplied.  No reference counterpart. */
T0B_API int32_t t0b_copy_d2d_async(t0b_ctx* ctx, uint64_t dst, size_t dst_pitch, uint64_t src, size_t src_pitch,
                                   size_t width_bytes, size_t rows);
/* The config t0b_gemm_multi_dst uses when it is given none: the auto_select tile for (m, k, n_local), except that
 * with peers a tile that keeps both TMEM accumulators for one tile (256x512, 512x256) becomes 256x256 -- whose
 * accumulators double-buffer, so that the peer stores of one tile retire while the next is multiplied -- once the
 * NVLink time of the stores exceeds half of the math time (four and eight GPUs on the benchmark shape; two GPUs keep
 * 256x512).  Never split-K.  No counterpart in the reference (single GPU). */
T0B_API int32_t t0b_multi_dst_config(uint32_t m, uint32_t k, uint32_t n_local, int32_t n_dst, int32_t num_sms,
                                     t0b_gemm_config* out);
/* Launch timeline (diagnostic; works in libt0b200_trace.so, the same sources built with -DT0B_TRACE by
 * `python -m t0_gpu_b200.build --trace`; the regular library returns T0B_ERR_UNSUPPORTED).  buf is a zeroed device
 * buffer of launches x T0B_TRACE_CTAS x 16 uint64; GEMM launch i of the context (tcgen05 kernels with at most
 * T0B_TRACE_CTAS CTAs) stamps %globaltimer nanoseconds into buf[i % launches][blockIdx.x][slot], one thread per role:
 * 0 kernel entry, 1 set-up done, 2 dependency wait returned, 3 first K block issued, 4 first operands arrived, 5 last
 * MMA issued, 6 accumulator complete, 7 last chunk staged, 8 stores complete, 9 teardown barrier, 10 all loads issued,
 * 12 / 13 cluster split-K: closing barrier passed / partials visible (otherwise clock64 at 4 and 5, so that cycles per
 * nanosecond gives the SM clock of the main loop), 14 TMEM freed.  buf = 0 stops the stamping.  `bench.py --workload
 * timeline` prints the phases.  The reference has no GPU timers at all (wall-clock Instant around dispatches,
 * src/t0/cost_model.rs:961-978). */
#define T0B_TRACE_CTAS 160
T0B_API int32_t t0b_trace_set(t0b_ctx* ctx, uint64_t buf, uint32_t launches);
/* Column-sharded GEMM with the all-gather folded into the epilogue: this rank computes C[:, col0 : col0+n_local]
 * and stores every finished tile into each of the n_dst row-major [M, ldc] destinations (its own and its
 * peers', as peer-mapped device pointers).  No counterpart in the reference (single GPU). */
T0B_API int32_t t0b_gemm_multi_dst(t0b_ctx* ctx, const t0b_gemm_config* cfg, int32_t trans_a, int32_t trans_b,
                                   uint64_t a, uint64_t b, const uint64_t* c_dsts, int32_t n_dst, uint32_t m,
                                   uint32_t n_local, uint32_t k, uint64_t lda, uint64_t ldb, uint64_t ldc,
                                   uint64_t col0, int32_t out_dtype, int32_t async);

/* The reference's split-K contract, unreduced: slab s (f32 [M,N], at y + s*M*N*4) receives the partial sum
 * of K chunk s; the caller reduces (src/t0/gemm_gen.rs:746-752; examples/test_gemm_correctness.rs:165-207).
 * NT layout, lda = ldb = k, as the 40-byte kernarg implies. */
T0B_API int32_t t0b_gemm_slabs(t0b_ctx* ctx, const t0b_gemm_config* cfg, uint64_t x, uint64_t wt, uint64_t y,
                               uint32_t m, uint32_t n, uint32_t k, uint32_t split_k, int32_t async);
/* Deterministic slab sum, s = 0..split_k-1 in order, starting from +0.0 (the order of
 * examples/test_gemm_correctness.rs:203-207), with optional fused epilogue / bf16 output. */
T0B_API int32_t t0b_splitk_reduce(t0b_ctx* ctx, uint64_t partial, uint32_t split_k, uint32_t m, uint32_t n,
                                  uint64_t slab_stride_elems, uint64_t ld_partial, uint64_t c, uint64_t ldc,
                                  int32_t out_dtype, int32_t epilogue, uint64_t bias, float alpha, int32_t async);

/* Drop-in for `queue.submit(&kernel, [gx, gy, 1], kernargs)` + optional wait (src/kfd/mod.rs:1290, 1571;
 * GpuRuntime::dispatch, gpu_context.rs:264-288): takes the reference's kernarg blob (40, 44 or 48 bytes) and
 * the thread grid compute_grid* returned.  The 40/48-byte blobs do not carry M: it is recovered from the
 * grid, M = tiles_m * tile_m, exact because that path requires tile-aligned shapes. Split-K blobs
 * (y_split_stride != 0) leave unreduced slabs in Y. */
T0B_API int32_t t0b_dispatch_kernargs(t0b_ctx* ctx, const t0b_gemm_config* cfg, uint32_t grid_x, uint32_t grid_y,
                                      const uint8_t* kernargs, size_t kernargs_len, int32_t async);

/* Measure the candidate configs for (M, N, K) on the device and return the fastest
 * (GemmTuner::tune(rt, m, n, k), src/t0/auto_gemm.rs:82-162 -- argument order (M, N, K)). */
T0B_API int32_t t0b_tune(t0b_ctx* ctx, uint32_t m, uint32_t n, uint32_t k, int32_t trans_a, int32_t trans_b,
                         int32_t out_dtype, t0b_gemm_config* best, float* best_tflops);

/* Autotune cache on disk, the reference's wire format (src/t0/auto_gemm.rs:325-391): one file
 * <dir>/gemm_<M>x<N>x<K>.json holding {"tile_m":..,"tile_n":..,"tile_k":..,"wg_size":..,"split_k":..,"lds_pad":..,
 * "n_col_passes":..,"wgp":bool,"swap":bool,"tflops":..,"all":[..]}.  dir NULL = $T0_AUTOTUNE_DIR, else
 * $HOME/.t0_autotune.  load returns T0B_ERR_INVALID when there is no (parsable) entry.  t0b_tune consults and
 * updates this cache when the context has a directory set with t0b_set_autotune_dir. */
T0B_API int32_t t0b_tune_cache_save(const char* dir, uint32_t m, uint32_t n, uint32_t k, const t0b_gemm_config* cfg,
                                    float tflops);
T0B_API int32_t t0b_tune_cache_load(const char* dir, uint32_t m, uint32_t n, uint32_t k, t0b_gemm_config* cfg,
                                    float* tflops);
/* GemmTuner::invalidate / clear (auto_gemm.rs:394-404). */
T0B_API int32_t t0b_tune_cache_invalidate(const char* dir, uint32_t m, uint32_t n, uint32_t k);
/* dir NULL = the default directory above; "" = stop consulting the disk cache (the state of a new context). */
T0B_API int32_t t0b_set_autotune_dir(t0b_ctx* ctx, const char* dir);

/* ------------------------------------------------------------------------------------------------
 * Element-wise and row kernels around the GEMMs (f32 activations)
 * ---------------------------------------------------------------------------------------------- */

/* bf16 weight cache: GpuRuntime::get_or_create_bf16 / invalidate_bf16 / clear_bf16_cache
 * (src/ignis/gpu_context.rs:392-432).  The first call for a tensor id converts the f32 buffer on the device
 * (stream-ordered, no synchronisation) and keeps the bf16 copy; later calls return the same copy until the id is
 * invalidated -- which the caller does after every update of the weights (an optimizer step).  The copies live in
 * the context's buffer pool.  t0b_bf16_cache_stats counts entries, conversions run and hits. */
T0B_API int32_t t0b_get_or_create_bf16(t0b_ctx* ctx, uint64_t tensor_id, uint64_t f32_ptr, size_t n_elems,
                                       uint64_t* bf16_ptr);
T0B_API int32_t t0b_invalidate_bf16(t0b_ctx* ctx, uint64_t tensor_id);
T0B_API int32_t t0b_clear_bf16_cache(t0b_ctx* ctx);
T0B_API int32_t t0b_bf16_cache_stats(t0b_ctx* ctx, uint64_t* entries, uint64_t* conversions, uint64_t* hits);

/* f32 -> bf16, round to nearest even (src/ignis/ops/bf16_matmul.rs:357-384, done on the host there). */
T0B_API int32_t t0b_cast_f32_to_bf16(t0b_ctx* ctx, uint64_t src, uint64_t dst, size_t n, int32_t async);
/* f32 [rows, cols] -> bf16 [cols, rows] (f32_to_bf16_transpose_gpu_padded, bf16_matmul.rs:390-424). */
T0B_API int32_t t0b_cast_f32_to_bf16_transpose(t0b_ctx* ctx, uint64_t src, uint64_t dst, uint32_t rows,
                                               uint32_t cols, int32_t async);
/* RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * weight; optionally saves inv_rms[row]
 * (src/t0/rmsnorm_kernels.rs:37-88, 140-153; src/ignis/ops/rmsnorm.rs:40-124). */
T0B_API int32_t t0b_rmsnorm_fwd(t0b_ctx* ctx, uint64_t x, uint64_t weight, uint64_t y, uint64_t inv_rms,
                                uint32_t rows, uint32_t cols, float eps, int32_t async);
/* RMSNorm backward: dx (rmsnorm_kernels.rs:90-137, 155-174) and, when dgamma != 0, dgamma[c] = sum_r dy*x*inv_rms
 * reduced in a fixed order (the reference uses unordered atomics, src/ignis/ops/rmsnorm.rs:239-293).
 * dgamma needs a scratch of t0b_rmsnorm_bwd_scratch_bytes(rows, cols). */
T0B_API int32_t t0b_rmsnorm_bwd(t0b_ctx* ctx, uint64_t dy, uint64_t x, uint64_t weight, uint64_t dx, uint64_t dgamma,
                                uint64_t scratch, size_t scratch_bytes, uint32_t rows, uint32_t cols, float eps,
                                int32_t async);
T0B_API size_t t0b_rmsnorm_bwd_scratch_bytes(uint32_t rows, uint32_t cols);
/* RMSNorm backward (dx and dgamma; the same values as t0b_rmsnorm_bwd up to the order of the fp32 sums, and bit for
 * bit the same where both take the same kernels: cols < 1024 or unaligned rows) for callers that cannot allocate device
 * memory -- a host runtime that handed its whole device budget to fixed buffers at start-up, or a step loop that
 * must avoid the device-wide synchronisation cudaMalloc / cudaFree bring -- and so have no scratch to pass.
 * Has no counterpart in the reference.  The dgamma scratch lives in a 2 MiB array inside the library image
 * (resident on every GPU that loads the library until the process exits); nothing is allocated or freed by this
 * call.  Limit: rows + 64 * cols <= 524288 floats (for example 1024 x 4096, or 8192 x 8064); larger problems are
 * rejected with T0B_ERR_INVALID and must use t0b_rmsnorm_bwd.  The first call on a device looks up the array's
 * device address; make that first call outside any stream capture.  All calls on one GPU share the array
 * (whatever the context or stream): two calls that overlap on the GPU race on it, so keep them ordered.  The
 * array keeps the previous call's contents; every value read is rewritten first, so no clearing is needed.
 * dx may be 0 (dgamma only). */
T0B_API int32_t t0b_rmsnorm_bwd_noalloc(t0b_ctx* ctx, uint64_t dy, uint64_t x, uint64_t weight, uint64_t dx,
                                        uint64_t dgamma, uint32_t rows, uint32_t cols, float eps, int32_t async);
/* Row softmax forward / backward, any column count (src/t0/softmax_kernels.rs:38-146; cols <= 256 there). */
T0B_API int32_t t0b_softmax_fwd(t0b_ctx* ctx, uint64_t x, uint64_t y, uint32_t rows, uint32_t cols, int32_t async);
T0B_API int32_t t0b_softmax_bwd(t0b_ctx* ctx, uint64_t dy, uint64_t y, uint64_t dx, uint32_t rows, uint32_t cols,
                                int32_t async);
/* Fused softmax cross-entropy: losses[r] = logsumexp(x_r) - x_r[target_r] and
 * dlogits = (softmax - onehot) * scale in one pass pair over the logits
 * (src/t0/ce_loss_kernels.rs:26-192; examples/kernels/softmax_ce_loss.rs:58-308). Either output may be 0. */
T0B_API int32_t t0b_softmax_ce(t0b_ctx* ctx, uint64_t logits, uint64_t targets_u32, uint64_t losses,
                               uint64_t dlogits, uint32_t rows, uint32_t cols, uint64_t ld, float scale,
                               int32_t async);
/* SiLU gate forward / backward (src/ignis/ops/silu.rs:32-152). up == 0 means plain SiLU (up = 1). */
T0B_API int32_t t0b_silu_gate_fwd(t0b_ctx* ctx, uint64_t gate, uint64_t up, uint64_t out, size_t n, int32_t async);
T0B_API int32_t t0b_silu_gate_bwd(t0b_ctx* ctx, uint64_t grad, uint64_t gate, uint64_t up, uint64_t dgate,
                                  uint64_t dup, size_t n, int32_t async);
/* y += x (grad accumulate; src/ignis/tape.rs:343-367, src/t0/elementwise_kernels.rs:41-61). */
T0B_API int32_t t0b_residual_add(t0b_ctx* ctx, uint64_t y, uint64_t x, size_t n, int32_t async);
/* Fused AdamW step (src/t0/adamw_kernels.rs:35-119); optionally refreshes a bf16 copy of the parameters. */
T0B_API int32_t t0b_adamw_step(t0b_ctx* ctx, uint64_t params, uint64_t grads, uint64_t m, uint64_t v,
                               uint64_t params_bf16, size_t n, float lr, float beta1, float beta2, float eps,
                               float weight_decay, uint32_t t, float grad_scale, int32_t async);

/* Fusions of the memory-bound steps between two GEMMs of the MLP (no single reference counterpart: the reference runs
 * each step as its own kernel, and lists such fusions as EpilogueOp chains, src/t0/tile_ir.rs:2213-2339).  Each gives
 * the same values as the sequence of calls it replaces, with the intermediate f32 arrays never written to memory.
 *   t0b_softmax_ce_bf16  = t0b_softmax_ce, then t0b_cast_f32_to_bf16 of the gradient (the operand of the dW and
 *                          dX GEMMs): dlogits is bf16[rows, ld].
 *   t0b_rmsnorm_silu_fwd = t0b_rmsnorm_fwd, t0b_silu_gate_fwd (no up operand), t0b_cast_f32_to_bf16:
 *                          out_bf16[rows, cols] = bf16(silu(rmsnorm(x))); inv_rms f32[rows] optional.
 *   t0b_rmsnorm_silu_bwd = t0b_silu_gate_bwd on the recomputed rmsnorm(x), t0b_rmsnorm_bwd, t0b_cast_f32_to_bf16:
 *                          dh f32 is the gradient of the SiLU output; dx_bf16 = bf16(d loss / d x); dgamma f32[cols]
 *                          optional, with scratch as for t0b_rmsnorm_bwd. */
T0B_API int32_t t0b_softmax_ce_bf16(t0b_ctx* ctx, uint64_t logits, uint64_t targets, uint64_t losses, uint64_t dlogits_bf16,
                                    uint32_t rows, uint32_t cols, uint64_t ld, float scale, int32_t async);
T0B_API int32_t t0b_rmsnorm_silu_fwd(t0b_ctx* ctx, uint64_t x, uint64_t weight, uint64_t out_bf16, uint64_t inv_rms,
                                     uint32_t rows, uint32_t cols, float eps, int32_t async);
T0B_API int32_t t0b_rmsnorm_silu_bwd(t0b_ctx* ctx, uint64_t dh, uint64_t x, uint64_t weight, uint64_t dx_bf16, uint64_t dgamma,
                                     uint64_t scratch, size_t scratch_bytes, uint32_t rows, uint32_t cols, float eps,
                                     int32_t async);

/* Embedding lookup and its gradient (src/t0/embedding_kernels.rs:30-96; Ignis: src/ignis/ops/embedding.rs:25-178).
 * table f32[vocab, dim], ids u32[num_tokens], out / grad_out f32[num_tokens, dim], any dim.
 *   fwd: out[t, :] = table[ids[t], :].
 *   bwd: grad_table[ids[t], :] += grad_out[t, :], rows of one id added in ascending token order (the order of the
 *        reference's CPU loop, :113-124), so the result is bit-identical to that loop and the same on every run; the
 *        reference's GPU kernel uses unordered float atomics.  grad_table is accumulated into (zero it first for a
 *        plain gradient, as the reference's caller does, embedding.rs:112-113).
 * An id >= vocab touches no memory: its output row is zeros (fwd) / it is skipped (bwd), and the device status word is
 * set to 110.  The backward sorts the token positions by id; scratch of t0b_embedding_bwd_scratch_bytes(num_tokens)
 * bytes (256-byte aligned) may be passed, or 0 to take it from the context's pool. */
T0B_API int32_t t0b_embedding_fwd(t0b_ctx* ctx, uint64_t table, uint64_t ids, uint64_t out, uint32_t num_tokens,
                                  uint32_t dim, uint32_t vocab, int32_t async);
T0B_API size_t t0b_embedding_bwd_scratch_bytes(uint32_t num_tokens);
T0B_API int32_t t0b_embedding_bwd(t0b_ctx* ctx, uint64_t grad_table, uint64_t ids, uint64_t grad_out, uint32_t num_tokens,
                                  uint32_t dim, uint32_t vocab, uint64_t scratch, size_t scratch_bytes, int32_t async);

/* ------------------------------------------------------------------------------------------------
 * tile_ir front end: TileGemm specs with M/N/K edge handling and an epilogue chain (src/t0/tile_ir.rs).
 * ---------------------------------------------------------------------------------------------- */
enum { T0B_TILE_NT = 0, T0B_TILE_NN = 1 };          /* TileTranspose, src/t0/tile_ir.rs:72-78 */
#define T0B_TILE_MAX_EPILOGUE 4
/* struct TileGemm, src/t0/tile_ir.rs:92-117.  `epilogue` holds T0B_EPI_* codes of the tile_ir members
 * (BIAS, SCALE, RELU, SILU, GELU_SIGMOID, ABS, NEG, CLAMP), applied in order. */
typedef struct t0b_tile_gemm {
    uint32_t tile_m, tile_n, tile_k;
    uint32_t wgp_mode, double_buffer;
    uint32_t split_k;                                /* 1 = none */
    uint32_t swap_grid;
    uint32_t transpose;                              /* T0B_TILE_NT / T0B_TILE_NN */
    uint32_t acc_swap;
    uint32_t n_epilogue;
    int32_t epilogue[T0B_TILE_MAX_EPILOGUE];
} t0b_tile_gemm;
/* The named constructors TileGemm::tile_*(), src/t0/tile_ir.rs:119-316: "128x64_k16", "64x64_k16", "64x64_k32",
 * "64x64_k64", "32x64_k16", "128x64_k32", "64x128_k32", "64x128_k16", "128x128_k16", "128x128_k32", "128x128_k48",
 * "128x128_k16_swap", "128x128_k32_swap", "256x64_k32_wgp", "256x64_k64_wgp", "128x128_k64", "128x64_k64". */
T0B_API int32_t t0b_tile_preset(const char* name, t0b_tile_gemm* out);
/* TileGemm::name(), src/t0/tile_ir.rs:406-433 (the kernel-cache key).  Returns the length written, <0 on error. */
T0B_API int32_t t0b_tile_name(const t0b_tile_gemm* spec, char* buf, size_t cap);
/* TileGemm::wg_size() / lds_total(), src/t0/tile_ir.rs:375-397. */
T0B_API uint32_t t0b_tile_wg_size(const t0b_tile_gemm* spec);
T0B_API uint32_t t0b_tile_lds_total(const t0b_tile_gemm* spec);
/* tile_auto_select(m, k, n, transpose), src/t0/tile_ir.rs:471-568: same branch outcomes (tile and split_k). */
T0B_API int32_t t0b_tile_auto_select(uint32_t m, uint32_t k, uint32_t n, uint32_t transpose, t0b_tile_gemm* out);
/* tile_ir::compute_grid, src/t0/tile_ir.rs:3193-3202: [x threads, y workgroups * split_k, 1]. */
T0B_API int32_t t0b_tile_compute_grid(const t0b_tile_gemm* spec, uint32_t m, uint32_t n, uint32_t grid[3]);
/* The kernarg blob of a lowered TileGemm: the 44 bytes of build_kernargs_m (src/t0/tile_ir.rs:3173-3190; the
 * split_k_shift field at 32..36 is filled from the spec) followed by the epilogue arguments in the order lower_gemm
 * declares them (src/t0/tile_ir.rs:670-682), each naturally aligned: bias pointer (u64, at 48) if the chain has
 * BiasAdd, scale (f32) if it has Scale, clamp_min and clamp_max (f32) if it has Clamp.  Returns the length written
 * (44..68), <0 on error. */
T0B_API int32_t t0b_tile_build_kernargs(const t0b_tile_gemm* spec, uint64_t x, uint64_t wt, uint64_t y, uint32_t k,
                                        uint32_t n, uint32_t m, uint64_t bias, float scale, float clamp_min,
                                        float clamp_max, uint8_t* out, size_t cap);
/* lower_gemm(&spec) + ensure_kernel_t0 + dispatch (src/t0/tile_ir.rs:585, src/ignis/gpu_context.rs:196-332) in one
 * call: runs the spec on the blob above.  NT reads WT[N,K] (pitch K), NN reads B[K,N] (pitch N); X has pitch K, Y
 * pitch N.  Any M, N, K (edges are masked; no padding needed).  `grid` must equal t0b_tile_compute_grid for the M in
 * the blob.  split_k > 1 produces the complete product in Y (slabs summed on the device in slab order); the
 * reference's tile_ir kernels leave y_split_stride at 0 there and race on Y (src/t0/cost_model.rs:570-571). */
T0B_API int32_t t0b_tile_dispatch(t0b_ctx* ctx, const t0b_tile_gemm* spec, const uint32_t grid[3], const uint8_t* kernargs,
                                  size_t len, int32_t async);

/* ------------------------------------------------------------------------------------------------
 * CUDA-graph capture for launch-bound shapes (takes the place of the AQL batch submit,
 * GpuRuntime::dispatch_async + wait_idle, gpu_context.rs:332, 297).
 * ---------------------------------------------------------------------------------------------- */
T0B_API int32_t t0b_graph_begin(t0b_ctx* ctx);
T0B_API int32_t t0b_graph_end(t0b_ctx* ctx, uint64_t* graph_handle);
T0B_API int32_t t0b_graph_launch(t0b_ctx* ctx, uint64_t graph_handle, int32_t async);
T0B_API int32_t t0b_graph_destroy(t0b_ctx* ctx, uint64_t graph_handle);

/* ------------------------------------------------------------------------------------------------
 * Diagnostics
 * ---------------------------------------------------------------------------------------------- */
/* Runs a one-thread kernel that waits on a barrier nobody signals; the wait runs out after limit_ns, the
 * kernel records its status code and returns.  Returns T0B_ERR_DEVICE and leaves the context usable. */
T0B_API int32_t t0b_selftest_bounded_wait(t0b_ctx* ctx, uint64_t limit_ns);
/* Time `iters` back-to-back launches of one GEMM with CUDA events on the context's stream; ms per launch. */
T0B_API int32_t t0b_gemm_time(t0b_ctx* ctx, const t0b_gemm_config* cfg, int32_t trans_a, int32_t trans_b, uint64_t a,
                              uint64_t b, uint64_t c, uint32_t m, uint32_t n, uint32_t k, uint64_t lda, uint64_t ldb,
                              uint64_t ldc, int32_t out_dtype, int32_t warmup, int32_t iters, float* ms_per_launch);
/* Number of kernels this context has launched so far. */
T0B_API uint64_t t0b_launch_count(t0b_ctx* ctx);
T0B_API const char* t0b_version(void);

#ifdef __cplusplus
}
#endif
#endif /* T0B200_H */
