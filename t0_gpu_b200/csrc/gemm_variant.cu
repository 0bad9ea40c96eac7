// One tile variant of the tcgen05 GEMM kernel family: compiled once per variant with
//   -DT0B_V_BN=.. -DT0B_V_CG=.. -DT0B_V_MT=.. -DT0B_V_ND=..
// (columns per accumulator, CTAs per tile, M sub-tiles, two N halves).
#if !defined(T0B_V_BN) || !defined(T0B_V_CG) || !defined(T0B_V_MT) || !defined(T0B_V_ND)
#error "compile with -DT0B_V_BN= -DT0B_V_CG= -DT0B_V_MT= -DT0B_V_ND="
#endif
#define T0B_VARIANT T0B_V_BN, T0B_V_CG, T0B_V_MT, T0B_V_ND
#include "gemm_launch.cuh"

namespace t0b {
template int32_t launch_variant<T0B_VARIANT>(t0b_ctx*, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const GemmParams&, int, int);
#if T0B_V_CG == 1 && T0B_V_MT == 1 && T0B_V_ND == 0
template int max_active_splitk_clusters<T0B_V_BN>(t0b_ctx*, int);   // lives beside the single-CTA variant it queries
#endif
}  // namespace t0b
