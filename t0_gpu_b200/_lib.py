"""ctypes binding of libt0b200.so.  Loads the in-tree build; there is no fallback of any kind: if the
library is missing the import fails with the build command to run."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libt0b200.so")


class GemmConfigC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "tile_m", "tile_n", "tile_k", "wg_size", "use_lds", "double_buffer", "split_k", "lds_pad", "n_col_passes",
        "swap_grid", "wgp_mode", "transpose", "epilogue")]


class GemmPlanC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "bm", "bn", "bk", "cta_group", "m_tiles", "n_tiles", "stages", "split_k", "kb_per_split", "use_tma", "grid", "smem_bytes")]


class TileGemmC(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "tile_m", "tile_n", "tile_k", "wgp_mode", "double_buffer", "split_k", "swap_grid", "transpose", "acc_swap",
        "n_epilogue")] + [("epilogue", C.c_int32 * 4)]


_u32, _u64, _i32, _sz, _f = C.c_uint32, C.c_uint64, C.c_int32, C.c_size_t, C.c_float
_ctx = C.c_void_p
_cfgp = C.POINTER(GemmConfigC)
_u8p = C.POINTER(C.c_uint8)
_u32p = C.POINTER(C.c_uint32)

# name -> (restype, argtypes); one entry per symbol include/t0b200.h declares.
SIGNATURES = {
    "t0b_config_preset": (_i32, [C.c_char_p, _cfgp]),
    "t0b_config_name": (_i32, [_cfgp, C.c_char_p, _sz]),
    "t0b_sweep_configs": (_i32, [_cfgp, _i32]),
    "t0b_standard_configs": (_i32, [_cfgp, _i32]),
    "t0b_config_lds_total": (_u32, [_cfgp]),
    "t0b_config_estimated_vgprs": (_u32, [_cfgp]),
    "t0b_config_is_feasible": (_i32, [_cfgp]),
    "t0b_auto_select": (_i32, [_u32, _u32, _u32, _cfgp]),
    "t0b_auto_select_source": (_i32, [_u32, _u32, _u32, _i32, _i32, _i32, _cfgp]),
    "t0b_auto_select_legacy": (_i32, [_u32, _u32, _u32, _cfgp]),
    "t0b_auto_select_backward_data": (_i32, [_u32, _u32, _u32, _cfgp]),
    "t0b_auto_select_backward_weight": (_i32, [_u32, _u32, _u32, _cfgp]),
    "t0b_compute_grid": (_i32, [_cfgp, _u32, _u32, _u32p, _u32p]),
    "t0b_compute_grid_split_k": (_i32, [_cfgp, _u32, _u32, _u32, _u32p, _u32p]),
    "t0b_compute_grid_auto": (_i32, [_cfgp, _u32, _u32, _u32p, _u32p]),
    "t0b_compute_grid_backward_data": (_i32, [_cfgp, _u32, _u32, _u32p, _u32p]),
    "t0b_compute_grid_backward_weight": (_i32, [_cfgp, _u32, _u32, _u32p, _u32p]),
    "t0b_build_kernargs": (_i32, [_u64, _u64, _u64, _u32, _u32, _u32, _cfgp, _u8p]),
    "t0b_build_kernargs_with_bias": (_i32, [_u64, _u64, _u64, _u32, _u32, _u32, _cfgp, _u64, _u8p]),
    "t0b_build_kernargs_m": (_i32, [_u64, _u64, _u64, _u32, _u32, _u32, _u8p]),
    "t0b_build_kernargs_backward_data": (_i32, [_u64, _u64, _u64, _u32, _u32, _u32, _cfgp, _u8p]),
    "t0b_build_kernargs_backward_weight": (_i32, [_u64, _u64, _u64, _u32, _u32, _u32, _cfgp, _u8p]),
    "t0b_resolve_plan": (_i32, [_cfgp, _u32, _u32, _u32, _i32, _i32, _u64, _u64, _i32, C.POINTER(GemmPlanC)]),
    "t0b_ctx_create": (_i32, [_i32, C.POINTER(_ctx)]),
    "t0b_ctx_destroy": (None, [_ctx]),
    "t0b_ctx_set_stream": (_i32, [_ctx, C.c_void_p]),
    "t0b_ctx_stream": (C.c_void_p, [_ctx]),
    "t0b_last_error": (C.c_char_p, [_ctx]),
    "t0b_is_poisoned": (_i32, [_ctx]),
    "t0b_num_sms": (_i32, [_ctx]),
    "t0b_set_sm_limit": (_i32, [_ctx, _i32]),
    "t0b_device_status": (_i32, [_ctx, _i32]),
    "t0b_set_wait_limit_ns": (_i32, [_ctx, _u64]),
    "t0b_alloc": (_i32, [_ctx, _sz, C.POINTER(_u64)]),
    "t0b_alloc_zero": (_i32, [_ctx, _sz, C.POINTER(_u64)]),
    "t0b_recycle": (_i32, [_ctx, _u64]),
    "t0b_free": (_i32, [_ctx, _u64]),
    "t0b_pool_stats": (_i32, [_ctx, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)]),
    "t0b_memcpy_h2d": (_i32, [_ctx, _u64, C.c_void_p, _sz]),
    "t0b_memcpy_d2h": (_i32, [_ctx, C.c_void_p, _u64, _sz]),
    "t0b_memset0": (_i32, [_ctx, _u64, _sz]),
    "t0b_memcpy2d_d2h": (_i32, [_ctx, C.c_void_p, _sz, _u64, _sz, _sz, _sz]),
    "t0b_memcpy_h2d_async": (_i32, [_ctx, _u64, C.c_void_p, _sz]),
    "t0b_memcpy2d_d2h_async": (_i32, [_ctx, C.c_void_p, _sz, _u64, _sz, _sz, _sz]),
    "t0b_sync": (_i32, [_ctx]),
    "t0b_ipc_export": (_i32, [_ctx, _u64, _u8p]),
    "t0b_ipc_open": (_i32, [_ctx, _u8p, C.POINTER(_u64)]),
    "t0b_ipc_close": (_i32, [_ctx, _u64]),
    "t0b_gemm": (_i32, [_ctx, _cfgp, _i32, _i32, _u64, _u64, _u64, _u32, _u32, _u32, _u64, _u64, _u64, _i32, _i32,
                        _u64, _f, _u64, _sz, _i32]),
    "t0b_gemm_chain": (_i32, [_ctx, _cfgp, _i32, _i32, _u64, _u64, _u64, _u32, _u32, _u32, _u64, _u64, _u64, _i32,
                              C.POINTER(_i32), _i32, _u64, _f, _f, _f, _u64, _sz, _i32]),
    "t0b_gemm_workspace_bytes": (_sz, [_cfgp, _u32, _u32, _u32]),
    "t0b_gemm_host": (_i32, [_ctx, _cfgp, _i32, _i32, C.c_void_p, C.c_void_p, C.c_void_p, _u32, _u32, _u32, _u64, _u64, _u64,
                             _i32, _u32]),
    "t0b_hash_blocks": (_i32, [_ctx, _u64, _sz, _sz, _u64, _i32]),
    "t0b_copy_d2d": (_i32, [_ctx, _u64, _sz, _u64, _sz, _sz, _sz, _i32]),
    "t0b_copy_d2d_async": (_i32, [_ctx, _u64, _sz, _u64, _sz, _sz, _sz]),
    "t0b_trace_set": (_i32, [_ctx, _u64, _u32]),
    "t0b_multi_dst_config": (_i32, [_u32, _u32, _u32, _i32, _i32, _cfgp]),
    "t0b_gemm_multi_dst": (_i32, [_ctx, _cfgp, _i32, _i32, _u64, _u64, C.POINTER(_u64), _i32, _u32, _u32, _u32, _u64,
                                  _u64, _u64, _u64, _i32, _i32]),
    "t0b_gemm_slabs": (_i32, [_ctx, _cfgp, _u64, _u64, _u64, _u32, _u32, _u32, _u32, _i32]),
    "t0b_splitk_reduce": (_i32, [_ctx, _u64, _u32, _u32, _u32, _u64, _u64, _u64, _u64, _i32, _i32, _u64, _f, _i32]),
    "t0b_dispatch_kernargs": (_i32, [_ctx, _cfgp, _u32, _u32, _u8p, _sz, _i32]),
    "t0b_softmax_ce_bf16": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u32, _u32, _u64, _f, _i32]),
    "t0b_rmsnorm_silu_fwd": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u32, _u32, _f, _i32]),
    "t0b_rmsnorm_silu_bwd": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u64, _u64, _sz, _u32, _u32, _f, _i32]),
    "t0b_embedding_fwd": (_i32, [_ctx, _u64, _u64, _u64, _u32, _u32, _u32, _i32]),
    "t0b_embedding_bwd_scratch_bytes": (_sz, [_u32]),
    "t0b_embedding_bwd": (_i32, [_ctx, _u64, _u64, _u64, _u32, _u32, _u32, _u64, _sz, _i32]),
    "t0b_tile_preset": (_i32, [C.c_char_p, C.POINTER(TileGemmC)]),
    "t0b_tile_name": (_i32, [C.POINTER(TileGemmC), C.c_char_p, _sz]),
    "t0b_tile_wg_size": (_u32, [C.POINTER(TileGemmC)]),
    "t0b_tile_lds_total": (_u32, [C.POINTER(TileGemmC)]),
    "t0b_tile_auto_select": (_i32, [_u32, _u32, _u32, _u32, C.POINTER(TileGemmC)]),
    "t0b_tile_compute_grid": (_i32, [C.POINTER(TileGemmC), _u32, _u32, _u32p]),
    "t0b_tile_build_kernargs": (_i32, [C.POINTER(TileGemmC), _u64, _u64, _u64, _u32, _u32, _u32, _u64, _f, _f, _f, _u8p, _sz]),
    "t0b_tile_dispatch": (_i32, [_ctx, C.POINTER(TileGemmC), _u32p, _u8p, _sz, _i32]),
    "t0b_tune": (_i32, [_ctx, _u32, _u32, _u32, _i32, _i32, _i32, _cfgp, C.POINTER(_f)]),
    "t0b_tune_cache_save": (_i32, [C.c_char_p, _u32, _u32, _u32, _cfgp, _f]),
    "t0b_tune_cache_load": (_i32, [C.c_char_p, _u32, _u32, _u32, _cfgp, C.POINTER(_f)]),
    "t0b_tune_cache_invalidate": (_i32, [C.c_char_p, _u32, _u32, _u32]),
    "t0b_set_autotune_dir": (_i32, [_ctx, C.c_char_p]),
    "t0b_get_or_create_bf16": (_i32, [_ctx, _u64, _u64, _sz, C.POINTER(_u64)]),
    "t0b_invalidate_bf16": (_i32, [_ctx, _u64]),
    "t0b_clear_bf16_cache": (_i32, [_ctx]),
    "t0b_bf16_cache_stats": (_i32, [_ctx, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)]),
    "t0b_cast_f32_to_bf16": (_i32, [_ctx, _u64, _u64, _sz, _i32]),
    "t0b_cast_f32_to_bf16_transpose": (_i32, [_ctx, _u64, _u64, _u32, _u32, _i32]),
    "t0b_rmsnorm_fwd": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u32, _u32, _f, _i32]),
    "t0b_rmsnorm_bwd": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u64, _u64, _sz, _u32, _u32, _f, _i32]),
    "t0b_rmsnorm_bwd_scratch_bytes": (_sz, [_u32, _u32]),
    "t0b_rmsnorm_bwd_noalloc": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u64, _u32, _u32, _f, _i32]),
    "t0b_softmax_fwd": (_i32, [_ctx, _u64, _u64, _u32, _u32, _i32]),
    "t0b_softmax_bwd": (_i32, [_ctx, _u64, _u64, _u64, _u32, _u32, _i32]),
    "t0b_softmax_ce": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u32, _u32, _u64, _f, _i32]),
    "t0b_silu_gate_fwd": (_i32, [_ctx, _u64, _u64, _u64, _sz, _i32]),
    "t0b_silu_gate_bwd": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u64, _sz, _i32]),
    "t0b_residual_add": (_i32, [_ctx, _u64, _u64, _sz, _i32]),
    "t0b_adamw_step": (_i32, [_ctx, _u64, _u64, _u64, _u64, _u64, _sz, _f, _f, _f, _f, _f, _u32, _f, _i32]),
    "t0b_graph_begin": (_i32, [_ctx]),
    "t0b_graph_end": (_i32, [_ctx, C.POINTER(_u64)]),
    "t0b_graph_launch": (_i32, [_ctx, _u64, _i32]),
    "t0b_graph_destroy": (_i32, [_ctx, _u64]),
    "t0b_selftest_bounded_wait": (_i32, [_ctx, _u64]),
    "t0b_gemm_time": (_i32, [_ctx, _cfgp, _i32, _i32, _u64, _u64, _u64, _u32, _u32, _u32, _u64, _u64, _u64, _i32, _i32,
                             _i32, C.POINTER(_f)]),
    "t0b_launch_count": (_u64, [_ctx]),
    "t0b_version": (C.c_char_p, []),
}

_LIB = None
TRACE_LIB_PATH = os.path.join(HERE, "lib", "libt0b200_trace.so")


def load_trace_lib() -> C.CDLL:
    """The timeline build of the library (`python -m t0_gpu_b200.build --trace`): the same entry points, with GEMM
    kernels that stamp their phase changes (t0b_trace_set).  A separate library with its own contexts."""
    if not os.path.exists(TRACE_LIB_PATH):
        raise ImportError(f"{TRACE_LIB_PATH} is missing: build it with `python -m t0_gpu_b200.build --trace`")
    L = C.CDLL(TRACE_LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m t0_gpu_b200.build` (needs nvcc); "
                "there is no CPU or PyTorch fallback for this library")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)   # AttributeError here = header/library mismatch
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB
