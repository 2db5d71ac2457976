// One instantiation of a tcgen05 GEMM kernel and its host launcher. The Makefile compiles this file once per
// variant with  -DINST_NAME=<launcher name> -DINST_KIND=<KIND_*> and either -DINST_PAIR_EPI=<1|2> -DINST_PAIR_CUT=<0|1>
// (CTA-pair kernel) or -DINST_BLOCK_N=<128|256> -DINST_STAGES=<n> (single-CTA kernel).
#include <cstring>

#include "gemm_launch.h"
#include "gemm_sm100_pair.cuh"

namespace mmeb200 {

#define INST_CAT2(a, b) a##b
#define INST_CAT(a, b) INST_CAT2(a, b)

#ifdef INST_PAIR_EPI

static int g_max_pairs[64] = {};

static LaunchResult configure(const LaunchEnv& env, int* pairs) {
    auto kern = gemm_tcgen05_pair_kernel<INST_KIND, INST_PAIR_EPI, INST_PAIR_CUT != 0>;
    constexpr int smem = PairSmem<INST_PAIR_EPI>::kTotal;
    constexpr int threads = PairSmem<INST_PAIR_EPI>::kThreads;
    int& cached = g_max_pairs[env.device & 63];
    if (cached == 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return {e, LAUNCH_OK, "cudaFuncSetAttribute(pair kernel)"};
        // a cluster needs both its SMs inside one GPC, so the device may hold fewer pairs than sm_count / 2
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof cfg);
        cfg.gridDim = dim3(unsigned(env.sm_count) & ~1u);
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess) return {e, LAUNCH_OK, "cudaOccupancyMaxActiveClusters(pair kernel)"};
        if (n <= 0) return {cudaSuccess, LAUNCH_NO_PAIR_FITS, "no CTA pair fits on this device"};
        cached = n;
    }
    *pairs = cached;
    return {cudaSuccess, LAUNCH_OK, ""};
}

int INST_CAT(INST_NAME, _capacity)(const LaunchEnv& env) {
    int n = 0;
    const LaunchResult r = configure(env, &n);
    return (r.cuda == cudaSuccess && r.code == LAUNCH_OK) ? n : 0;
}

LaunchResult INST_NAME(const LaunchEnv& env, const GemmParams& p, uint64_t tiles) {
    int cap = 0;
    const LaunchResult r = configure(env, &cap);
    if (r.cuda != cudaSuccess || r.code != LAUNCH_OK) return r;
    constexpr int smem = PairSmem<INST_PAIR_EPI>::kTotal;
    constexpr int threads = PairSmem<INST_PAIR_EPI>::kThreads;
    const unsigned pairs = unsigned(tiles < uint64_t(cap) ? tiles : uint64_t(cap));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(pairs * 2);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = env.stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = env.dependent_launch ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<INST_KIND, INST_PAIR_EPI, INST_PAIR_CUT != 0>, p);
    return {e != cudaSuccess ? e : cudaGetLastError(), LAUNCH_OK, "pair kernel launch"};
}

#else

static bool g_configured[64] = {};

LaunchResult INST_NAME(const LaunchEnv& env, const GemmParams& p, unsigned grid) {
    auto kern = gemm_tcgen05_kernel<INST_KIND, INST_BLOCK_N, INST_STAGES>;
    constexpr int smem = GemmSmem<INST_BLOCK_N, INST_STAGES>::kTotal;
    if (!g_configured[env.device & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return {e, LAUNCH_OK, "cudaFuncSetAttribute(gemm kernel)"};
        g_configured[env.device & 63] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = env.stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = env.dependent_launch ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    return {e != cudaSuccess ? e : cudaGetLastError(), LAUNCH_OK, "gemm kernel launch"};
}

#endif

}  // namespace mmeb200
