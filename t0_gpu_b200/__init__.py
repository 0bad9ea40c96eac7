"""t0_gpu_b200 -- B200 (sm_100a) implementation of T0-GPU's bf16 GEMM hot path.

The product is the C-ABI CUDA library (include/t0b200.h, built to t0_gpu_b200/lib/libt0b200.so); this
package is the thin host-side mirror of the reference interface over it.  Importing the package does not
load the library; the first call does, and fails loudly when it has not been built."""
from .gemm_gen import (EpilogueOp, GemmConfig, GemmPlan, GemmTranspose, auto_select, auto_select_backward_data,  # noqa: F401
                       auto_select_backward_weight, auto_select_legacy, auto_select_source, build_kernargs, build_kernargs_backward_data,
                       build_kernargs_backward_weight, build_kernargs_m, build_kernargs_with_bias, compute_grid,
                       compute_grid_auto, compute_grid_backward_data, compute_grid_backward_weight,
                       compute_grid_split_k, resolve_plan, standard_configs, sweep_configs)
from . import tile_ir  # noqa: F401
from .auto_gemm import GemmTuner, GemmTuneResult, auto_gemm, global_tuner  # noqa: F401
from .gpu_context import OUT_BF16, OUT_F32, GpuBuffer, GpuRuntime, T0Error  # noqa: F401
