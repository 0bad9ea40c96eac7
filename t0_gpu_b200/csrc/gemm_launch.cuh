// Launch wrapper of the GEMM kernel family, one instantiation per tile variant.  The variants are compiled in
// separate translation units (gemm_variant.cu, once per variant) so they build side by side; every other file
// sees them as extern templates.
#pragma once
#include <algorithm>
#include <mutex>

#include "gemm_sm100.cuh"
#include "t0b_internal.hpp"

namespace t0b {

template <int BN, int CG, int MT, int ND = 0>
int32_t launch_variant(t0b_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                       const GemmParams& p, int num_work, int cluster_sk = 0) {
    using T = GemmTraits<BN, CG, MT, ND>;
    auto kfn = gemm_bf16_tcgen05_kernel<BN, CG, MT, ND>;
    static bool configured[64] = {};
    static int max_clusters[64] = {};
    static std::mutex config_mu;   // several contexts (threads) may launch the same variant for the first time at once
    const int dev = ctx->device & 63;
    std::unique_lock<std::mutex> config_lock(config_mu);
    if (!configured[dev]) {
        int32_t rc = check_cuda(ctx, cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes),
                                "cudaFuncSetAttribute(smem)");
        if (rc != T0B_OK) return rc;
        if (CG == 2) {
            rc = check_cuda(ctx, cudaFuncSetAttribute(kfn, cudaFuncAttributeNonPortableClusterSizeAllowed, 0),
                            "cudaFuncSetAttribute(cluster)");
            if (rc != T0B_OK) return rc;
            cudaLaunchConfig_t qc{};
            qc.gridDim = dim3(ctx->num_sms - (ctx->num_sms % 2), 1, 1);
            qc.blockDim = dim3(T::kThreads, 1, 1);
            qc.dynamicSmemBytes = T::kSmemBytes;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension;
            qa[0].val.clusterDim.x = 2;
            qa[0].val.clusterDim.y = 1;
            qa[0].val.clusterDim.z = 1;
            qc.attrs = qa;
            qc.numAttrs = 1;
            int nc = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&nc, kfn, &qc);
            if (e != cudaSuccess || nc <= 0) {
                cudaGetLastError();
                nc = ctx->num_sms / 2;
            }
            max_clusters[dev] = nc;
        } else {
            max_clusters[dev] = ctx->num_sms;
        }
        configured[dev] = true;
    }
    int avail = max_clusters[dev];
    config_lock.unlock();
    if (ctx->sm_limit > 0) avail = std::min(avail, std::max(1, ctx->sm_limit / CG));   // leave SMs to concurrent kernels
    int clusters = std::max(1, std::min(num_work, avail));
    // Cluster split-K: one CTA per work item (not persistent), clusters of `cluster_sk` consecutive CTAs; the hardware
    // schedules whole clusters, so the K ranges of a tile always run together whatever the number of waves.
    if (cluster_sk > 1) clusters = num_work;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(clusters * CG, 1, 1);
    cfg.blockDim = dim3(T::kThreads, 1, 1);
    cfg.dynamicSmemBytes = T::kSmemBytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = cluster_sk > 1 ? cluster_sk : CG;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    // The kernel's set-up (barriers, TMEM allocation) overlaps the tail of the previous kernel in the stream; the
    // kernel itself waits (griddepcontrol.wait) before its first access to global memory.
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    return check_cuda(ctx, cudaLaunchKernelEx(&cfg, kfn, ta, tb, tc, p), "cudaLaunchKernelEx(gemm)");
}

// How many clusters of `cluster_sk` CTAs of a single-CTA variant can be resident at once on this device (GPC sizes
// bound it: eight-CTA clusters do not tile every GPC).  Cached per device and cluster size.
template <int BN>
int max_active_splitk_clusters(t0b_ctx* ctx, int cluster_sk) {
    using T = GemmTraits<BN, 1, 1, 0>;
    static int cache[64][9] = {};
    static std::mutex cache_mu;
    const int dev = ctx->device & 63;
    if (cluster_sk < 2 || cluster_sk > 8) return 0;
    std::lock_guard<std::mutex> lk(cache_mu);
    if (cache[dev][cluster_sk] != 0) return cache[dev][cluster_sk];
    auto kfn = gemm_bf16_tcgen05_kernel<BN, 1, 1, 0>;
    cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
    cudaLaunchConfig_t qc{};
    qc.gridDim = dim3(static_cast<unsigned>(cluster_sk * 64), 1, 1);
    qc.blockDim = dim3(T::kThreads, 1, 1);
    qc.dynamicSmemBytes = T::kSmemBytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = static_cast<unsigned>(cluster_sk);
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    qc.attrs = qa;
    qc.numAttrs = 1;
    int nc = 0;
    if (cudaOccupancyMaxActiveClusters(&nc, kfn, &qc) != cudaSuccess || nc <= 0) {
        cudaGetLastError();
        nc = ctx->num_sms / cluster_sk / 2;   // a cautious guess
    }
    cache[dev][cluster_sk] = nc;
    return nc;
}

#define T0B_GEMM_VARIANTS(X) X(256, 2, 2, 1) X(256, 2, 2, 0) X(256, 2, 1, 0) X(128, 2, 1, 0) X(256, 1, 1, 0) X(128, 1, 1, 0) X(64, 1, 1, 0)
#ifndef T0B_VARIANT
extern template int max_active_splitk_clusters<256>(t0b_ctx*, int);
extern template int max_active_splitk_clusters<128>(t0b_ctx*, int);
extern template int max_active_splitk_clusters<64>(t0b_ctx*, int);
#define T0B_EXTERN_VARIANT(BN, CG, MT, ND)                                                                              \
    extern template int32_t launch_variant<BN, CG, MT, ND>(t0b_ctx*, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, \
                                                            const GemmParams&, int, int);
T0B_GEMM_VARIANTS(T0B_EXTERN_VARIANT)
#undef T0B_EXTERN_VARIANT
#endif

}  // namespace t0b
