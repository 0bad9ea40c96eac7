// Generated from include/t0b200.h by include/make_sys_rs.py -- do not edit.
// The `-sys` layer of the B200 backend: `extern "C"` declarations of libt0b200.so, one per exported function.
#![allow(non_camel_case_types, dead_code)]
use std::os::raw::{c_char, c_void};

pub const T0B_OK: i32 = 0;
pub const T0B_ERR_INVALID: i32 = -1;
pub const T0B_ERR_CUDA: i32 = -2;
pub const T0B_ERR_POISONED: i32 = -3;
pub const T0B_ERR_DEVICE: i32 = -4;
pub const T0B_ERR_NOMEM: i32 = -5;
pub const T0B_ERR_UNSUPPORTED: i32 = -6;
pub const T0B_TRANSPOSE_NT: i32 = 0;
pub const T0B_TRANSPOSE_NN: i32 = 1;
pub const T0B_EPI_STORE_F32: i32 = 0;
pub const T0B_EPI_BIAS_ADD: i32 = 1;
pub const T0B_EPI_BIAS_ADD_RELU: i32 = 2;
pub const T0B_EPI_RELU: i32 = 3;
pub const T0B_EPI_SILU: i32 = 4;
pub const T0B_EPI_GELU_SIGMOID: i32 = 5;
pub const T0B_EPI_SCALE: i32 = 6;
pub const T0B_EPI_ABS: i32 = 7;
pub const T0B_EPI_NEG: i32 = 8;
pub const T0B_EPI_CLAMP: i32 = 9;
pub const T0B_OUT_F32: i32 = 0;
pub const T0B_OUT_BF16: i32 = 1;
pub const T0B_TILE_NT: i32 = 0;
pub const T0B_TILE_NN: i32 = 1;

#[repr(C)] pub struct t0b_ctx { _private: [u8; 0] }

#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct t0b_gemm_config {
    pub tile_m: u32,
    pub tile_n: u32,
    pub tile_k: u32,
    pub wg_size: u32,
    pub use_lds: u32,
    pub double_buffer: u32,
    pub split_k: u32,
    pub lds_pad: u32,
    pub n_col_passes: u32,
    pub swap_grid: u32,
    pub wgp_mode: u32,
    pub transpose: u32,
    pub epilogue: u32,
}

#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct t0b_gemm_plan {
    pub bm: u32,
    pub bn: u32,
    pub bk: u32,
    pub cta_group: u32,
    pub m_tiles: u32,
    pub n_tiles: u32,
    pub stages: u32,
    pub split_k: u32,
    pub kb_per_split: u32,
    pub use_tma: u32,
    pub grid: u32,
    pub smem_bytes: u32,
}

#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct t0b_tile_gemm {
    pub tile_m: u32,
    pub tile_n: u32,
    pub tile_k: u32,
    pub wgp_mode: u32,
    pub double_buffer: u32,
    pub split_k: u32,
    pub swap_grid: u32,
    pub transpose: u32,
    pub acc_swap: u32,
    pub n_epilogue: u32,
    pub epilogue[T0B_TILE_MAX_EPILOGUE]: i32,
}

extern "C" {
    pub fn t0b_config_preset(name: *const c_char, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_config_name(cfg: *const t0b_gemm_config, buf: *mut c_char, cap: usize) -> i32;
    pub fn t0b_sweep_configs(out: *mut t0b_gemm_config, cap: i32) -> i32;
    pub fn t0b_standard_configs(out: *mut t0b_gemm_config, cap: i32) -> i32;
    pub fn t0b_config_lds_total(cfg: *const t0b_gemm_config) -> u32;
    pub fn t0b_config_estimated_vgprs(cfg: *const t0b_gemm_config) -> u32;
    pub fn t0b_config_is_feasible(cfg: *const t0b_gemm_config) -> i32;
    pub fn t0b_auto_select(m: u32, k: u32, n: u32, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_auto_select_source(m: u32, k: u32, n: u32, trans_a: i32, trans_b: i32, out_dtype: i32, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_auto_select_legacy(m: u32, k: u32, n: u32, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_auto_select_backward_data(m: u32, n_orig: u32, k_orig: u32, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_auto_select_backward_weight(m: u32, n_orig: u32, k_orig: u32, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_compute_grid(cfg: *const t0b_gemm_config, m: u32, n: u32, gx: *mut u32, gy: *mut u32) -> i32;
    pub fn t0b_compute_grid_split_k(cfg: *const t0b_gemm_config, m: u32, n: u32, split_k: u32, gx: *mut u32, gy: *mut u32) -> i32;
    pub fn t0b_compute_grid_auto(cfg: *const t0b_gemm_config, m: u32, n: u32, gx: *mut u32, gy: *mut u32) -> i32;
    pub fn t0b_compute_grid_backward_data(cfg: *const t0b_gemm_config, m: u32, k_orig: u32, gx: *mut u32, gy: *mut u32) -> i32;
    pub fn t0b_compute_grid_backward_weight(cfg: *const t0b_gemm_config, n_orig: u32, k_orig: u32, gx: *mut u32, gy: *mut u32) -> i32;
    pub fn t0b_build_kernargs(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, cfg: *const t0b_gemm_config, out: *mut u8) -> i32;
    pub fn t0b_build_kernargs_with_bias(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, cfg: *const t0b_gemm_config, bias: u64, out: *mut u8) -> i32;
    pub fn t0b_build_kernargs_m(x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, out: *mut u8) -> i32;
    pub fn t0b_build_kernargs_backward_data(dy: u64, w: u64, dx: u64, m: u32, n_orig: u32, k_orig: u32, cfg: *const t0b_gemm_config, out: *mut u8) -> i32;
    pub fn t0b_build_kernargs_backward_weight(dy_t: u64, x_t: u64, dw: u64, m: u32, n_orig: u32, k_orig: u32, cfg: *const t0b_gemm_config, out: *mut u8) -> i32;
    pub fn t0b_resolve_plan(cfg: *const t0b_gemm_config, m: u32, n: u32, k: u32, trans_a: i32, trans_b: i32, lda: u64, ldb: u64, num_sms: i32, out: *mut t0b_gemm_plan) -> i32;
    pub fn t0b_ctx_create(device: i32, out: *mut *mut t0b_ctx) -> i32;
    pub fn t0b_ctx_destroy(ctx: *mut t0b_ctx);
    pub fn t0b_ctx_set_stream(ctx: *mut t0b_ctx, cuda_stream: *mut c_void) -> i32;
    pub fn t0b_ctx_stream(ctx: *mut t0b_ctx) -> *mut c_void;
    pub fn t0b_last_error(ctx: *mut t0b_ctx) -> *const c_char;
    pub fn t0b_is_poisoned(ctx: *mut t0b_ctx) -> i32;
    pub fn t0b_num_sms(ctx: *mut t0b_ctx) -> i32;
    pub fn t0b_set_sm_limit(ctx: *mut t0b_ctx, sms: i32) -> i32;
    pub fn t0b_device_status(ctx: *mut t0b_ctx, clear: i32) -> i32;
    pub fn t0b_set_wait_limit_ns(ctx: *mut t0b_ctx, ns: u64) -> i32;
    pub fn t0b_alloc(ctx: *mut t0b_ctx, bytes: usize, dptr: *mut u64) -> i32;
    pub fn t0b_alloc_zero(ctx: *mut t0b_ctx, bytes: usize, dptr: *mut u64) -> i32;
    pub fn t0b_recycle(ctx: *mut t0b_ctx, dptr: u64) -> i32;
    pub fn t0b_free(ctx: *mut t0b_ctx, dptr: u64) -> i32;
    pub fn t0b_pool_stats(ctx: *mut t0b_ctx, cached_bytes: *mut u64, hits: *mut u64, misses: *mut u64) -> i32;
    pub fn t0b_memcpy_h2d(ctx: *mut t0b_ctx, dst: u64, src: *const c_void, bytes: usize) -> i32;
    pub fn t0b_memcpy_d2h(ctx: *mut t0b_ctx, dst: *mut c_void, src: u64, bytes: usize) -> i32;
    pub fn t0b_memset0(ctx: *mut t0b_ctx, dst: u64, bytes: usize) -> i32;
    pub fn t0b_memcpy2d_d2h(ctx: *mut t0b_ctx, dst: *mut c_void, dst_pitch: usize, src: u64, src_pitch: usize, width_bytes: usize, height: usize) -> i32;
    pub fn t0b_memcpy_h2d_async(ctx: *mut t0b_ctx, dst: u64, src: *const c_void, bytes: usize) -> i32;
    pub fn t0b_memcpy2d_d2h_async(ctx: *mut t0b_ctx, dst: *mut c_void, dst_pitch: usize, src: u64, src_pitch: usize, width_bytes: usize, height: usize) -> i32;
    pub fn t0b_sync(ctx: *mut t0b_ctx) -> i32;
    pub fn t0b_ipc_export(ctx: *mut t0b_ctx, dptr: u64, handle: *mut u8) -> i32;
    pub fn t0b_ipc_open(ctx: *mut t0b_ctx, handle: *const u8, dptr: *mut u64) -> i32;
    pub fn t0b_ipc_close(ctx: *mut t0b_ctx, dptr: u64) -> i32;
    pub fn t0b_gemm(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, trans_a: i32, trans_b: i32, a: u64, b: u64, c: u64, m: u32, n: u32, k: u32, lda: u64, ldb: u64, ldc: u64, out_dtype: i32, epilogue: i32, bias: u64, alpha: f32, workspace: u64, workspace_bytes: usize, is_async: i32) -> i32;
    pub fn t0b_gemm_chain(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, trans_a: i32, trans_b: i32, a: u64, b: u64, c: u64, m: u32, n: u32, k: u32, lda: u64, ldb: u64, ldc: u64, out_dtype: i32, ops: *const i32, n_ops: i32, bias: u64, scale: f32, clamp_min: f32, clamp_max: f32, workspace: u64, workspace_bytes: usize, is_async: i32) -> i32;
    pub fn t0b_gemm_workspace_bytes(cfg: *const t0b_gemm_config, m: u32, n: u32, k: u32) -> usize;
    pub fn t0b_gemm_host(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, trans_a: i32, trans_b: i32, a: *const c_void, b: *const c_void, c: *mut c_void, m: u32, n: u32, k: u32, lda: u64, ldb: u64, ldc: u64, out_dtype: i32, chunk_rows: u32) -> i32;
    pub fn t0b_hash_blocks(ctx: *mut t0b_ctx, src: u64, bytes: usize, block_bytes: usize, out: u64, is_async: i32) -> i32;
    pub fn t0b_copy_d2d(ctx: *mut t0b_ctx, dst: u64, dst_pitch: usize, src: u64, src_pitch: usize, width_bytes: usize, rows: usize, is_async: i32) -> i32;
    pub fn t0b_copy_d2d_async(ctx: *mut t0b_ctx, dst: u64, dst_pitch: usize, src: u64, src_pitch: usize, width_bytes: usize, rows: usize) -> i32;
    pub fn t0b_multi_dst_config(m: u32, k: u32, n_local: u32, n_dst: i32, num_sms: i32, out: *mut t0b_gemm_config) -> i32;
    pub fn t0b_trace_set(ctx: *mut t0b_ctx, buf: u64, launches: u32) -> i32;
    pub fn t0b_gemm_multi_dst(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, trans_a: i32, trans_b: i32, a: u64, b: u64, c_dsts: *const u64, n_dst: i32, m: u32, n_local: u32, k: u32, lda: u64, ldb: u64, ldc: u64, col0: u64, out_dtype: i32, is_async: i32) -> i32;
    pub fn t0b_gemm_slabs(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, x: u64, wt: u64, y: u64, m: u32, n: u32, k: u32, split_k: u32, is_async: i32) -> i32;
    pub fn t0b_splitk_reduce(ctx: *mut t0b_ctx, partial: u64, split_k: u32, m: u32, n: u32, slab_stride_elems: u64, ld_partial: u64, c: u64, ldc: u64, out_dtype: i32, epilogue: i32, bias: u64, alpha: f32, is_async: i32) -> i32;
    pub fn t0b_dispatch_kernargs(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, grid_x: u32, grid_y: u32, kernargs: *const u8, kernargs_len: usize, is_async: i32) -> i32;
    pub fn t0b_tune(ctx: *mut t0b_ctx, m: u32, n: u32, k: u32, trans_a: i32, trans_b: i32, out_dtype: i32, best: *mut t0b_gemm_config, best_tflops: *mut f32) -> i32;
    pub fn t0b_tune_cache_save(dir: *const c_char, m: u32, n: u32, k: u32, cfg: *const t0b_gemm_config, tflops: f32) -> i32;
    pub fn t0b_tune_cache_load(dir: *const c_char, m: u32, n: u32, k: u32, cfg: *mut t0b_gemm_config, tflops: *mut f32) -> i32;
    pub fn t0b_tune_cache_invalidate(dir: *const c_char, m: u32, n: u32, k: u32) -> i32;
    pub fn t0b_set_autotune_dir(ctx: *mut t0b_ctx, dir: *const c_char) -> i32;
    pub fn t0b_get_or_create_bf16(ctx: *mut t0b_ctx, tensor_id: u64, f32_ptr: u64, n_elems: usize, bf16_ptr: *mut u64) -> i32;
    pub fn t0b_invalidate_bf16(ctx: *mut t0b_ctx, tensor_id: u64) -> i32;
    pub fn t0b_clear_bf16_cache(ctx: *mut t0b_ctx) -> i32;
    pub fn t0b_bf16_cache_stats(ctx: *mut t0b_ctx, entries: *mut u64, conversions: *mut u64, hits: *mut u64) -> i32;
    pub fn t0b_cast_f32_to_bf16(ctx: *mut t0b_ctx, src: u64, dst: u64, n: usize, is_async: i32) -> i32;
    pub fn t0b_cast_f32_to_bf16_transpose(ctx: *mut t0b_ctx, src: u64, dst: u64, rows: u32, cols: u32, is_async: i32) -> i32;
    pub fn t0b_rmsnorm_fwd(ctx: *mut t0b_ctx, x: u64, weight: u64, y: u64, inv_rms: u64, rows: u32, cols: u32, eps: f32, is_async: i32) -> i32;
    pub fn t0b_rmsnorm_bwd(ctx: *mut t0b_ctx, dy: u64, x: u64, weight: u64, dx: u64, dgamma: u64, scratch: u64, scratch_bytes: usize, rows: u32, cols: u32, eps: f32, is_async: i32) -> i32;
    pub fn t0b_rmsnorm_bwd_scratch_bytes(rows: u32, cols: u32) -> usize;
    pub fn t0b_rmsnorm_bwd_noalloc(ctx: *mut t0b_ctx, dy: u64, x: u64, weight: u64, dx: u64, dgamma: u64, rows: u32, cols: u32, eps: f32, is_async: i32) -> i32;
    pub fn t0b_softmax_fwd(ctx: *mut t0b_ctx, x: u64, y: u64, rows: u32, cols: u32, is_async: i32) -> i32;
    pub fn t0b_softmax_bwd(ctx: *mut t0b_ctx, dy: u64, y: u64, dx: u64, rows: u32, cols: u32, is_async: i32) -> i32;
    pub fn t0b_softmax_ce(ctx: *mut t0b_ctx, logits: u64, targets_u32: u64, losses: u64, dlogits: u64, rows: u32, cols: u32, ld: u64, scale: f32, is_async: i32) -> i32;
    pub fn t0b_silu_gate_fwd(ctx: *mut t0b_ctx, gate: u64, up: u64, out: u64, n: usize, is_async: i32) -> i32;
    pub fn t0b_silu_gate_bwd(ctx: *mut t0b_ctx, grad: u64, gate: u64, up: u64, dgate: u64, dup: u64, n: usize, is_async: i32) -> i32;
    pub fn t0b_residual_add(ctx: *mut t0b_ctx, y: u64, x: u64, n: usize, is_async: i32) -> i32;
    pub fn t0b_adamw_step(ctx: *mut t0b_ctx, params: u64, grads: u64, m: u64, v: u64, params_bf16: u64, n: usize, lr: f32, beta1: f32, beta2: f32, eps: f32, weight_decay: f32, t: u32, grad_scale: f32, is_async: i32) -> i32;
    pub fn t0b_softmax_ce_bf16(ctx: *mut t0b_ctx, logits: u64, targets: u64, losses: u64, dlogits_bf16: u64, rows: u32, cols: u32, ld: u64, scale: f32, is_async: i32) -> i32;
    pub fn t0b_rmsnorm_silu_fwd(ctx: *mut t0b_ctx, x: u64, weight: u64, out_bf16: u64, inv_rms: u64, rows: u32, cols: u32, eps: f32, is_async: i32) -> i32;
    pub fn t0b_rmsnorm_silu_bwd(ctx: *mut t0b_ctx, dh: u64, x: u64, weight: u64, dx_bf16: u64, dgamma: u64, scratch: u64, scratch_bytes: usize, rows: u32, cols: u32, eps: f32, is_async: i32) -> i32;
    pub fn t0b_embedding_fwd(ctx: *mut t0b_ctx, table: u64, ids: u64, out: u64, num_tokens: u32, dim: u32, vocab: u32, is_async: i32) -> i32;
    pub fn t0b_embedding_bwd_scratch_bytes(num_tokens: u32) -> usize;
    pub fn t0b_embedding_bwd(ctx: *mut t0b_ctx, grad_table: u64, ids: u64, grad_out: u64, num_tokens: u32, dim: u32, vocab: u32, scratch: u64, scratch_bytes: usize, is_async: i32) -> i32;
    pub fn t0b_tile_preset(name: *const c_char, out: *mut t0b_tile_gemm) -> i32;
    pub fn t0b_tile_name(spec: *const t0b_tile_gemm, buf: *mut c_char, cap: usize) -> i32;
    pub fn t0b_tile_wg_size(spec: *const t0b_tile_gemm) -> u32;
    pub fn t0b_tile_lds_total(spec: *const t0b_tile_gemm) -> u32;
    pub fn t0b_tile_auto_select(m: u32, k: u32, n: u32, transpose: u32, out: *mut t0b_tile_gemm) -> i32;
    pub fn t0b_tile_compute_grid(spec: *const t0b_tile_gemm, m: u32, n: u32, grid: *mut u32) -> i32;
    pub fn t0b_tile_build_kernargs(spec: *const t0b_tile_gemm, x: u64, wt: u64, y: u64, k: u32, n: u32, m: u32, bias: u64, scale: f32, clamp_min: f32, clamp_max: f32, out: *mut u8, cap: usize) -> i32;
    pub fn t0b_tile_dispatch(ctx: *mut t0b_ctx, spec: *const t0b_tile_gemm, grid: *const u32, kernargs: *const u8, len: usize, is_async: i32) -> i32;
    pub fn t0b_graph_begin(ctx: *mut t0b_ctx) -> i32;
    pub fn t0b_graph_end(ctx: *mut t0b_ctx, graph_handle: *mut u64) -> i32;
    pub fn t0b_graph_launch(ctx: *mut t0b_ctx, graph_handle: u64, is_async: i32) -> i32;
    pub fn t0b_graph_destroy(ctx: *mut t0b_ctx, graph_handle: u64) -> i32;
    pub fn t0b_selftest_bounded_wait(ctx: *mut t0b_ctx, limit_ns: u64) -> i32;
    pub fn t0b_gemm_time(ctx: *mut t0b_ctx, cfg: *const t0b_gemm_config, trans_a: i32, trans_b: i32, a: u64, b: u64, c: u64, m: u32, n: u32, k: u32, lda: u64, ldb: u64, ldc: u64, out_dtype: i32, warmup: i32, iters: i32, ms_per_launch: *mut f32) -> i32;
    pub fn t0b_launch_count(ctx: *mut t0b_ctx) -> u64;
    pub fn t0b_version() -> *const c_char;
}
