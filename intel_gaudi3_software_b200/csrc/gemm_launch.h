// Host-side launchers of the tcgen05 GEMM kernels. Every kernel instantiation is compiled in a
// translation unit of its own (gemm_inst.cu, built once per variant by the Makefile) so that the
// library builds in parallel; this header is what the planner in api.cu sees of them.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "gemm_sm100.cuh"

namespace mmeb200 {

struct LaunchEnv {
    int device;
    int sm_count;
    cudaStream_t stream;
    bool dependent_launch;   // launch with programmatic stream serialisation (set-up overlaps the previous kernel's tail)
};

enum : int { LAUNCH_OK = 0, LAUNCH_NO_PAIR_FITS = -1 };

// Result of a launch: cuda != cudaSuccess names the failing runtime call; code is one of LAUNCH_*.
struct LaunchResult {
    cudaError_t cuda;
    int code;
    const char* what;
};

// Single-CTA kernel, tile 128 x BLOCK_N (BLOCK_N = 256 with 4 stages, 128 with 6 stages).
LaunchResult launch_gemm_single(const LaunchEnv& env, uint32_t kind, int block_n, const GemmParams& p, unsigned grid);
// CTA-pair kernel, tile 256 x 256, with one or two groups of four epilogue warps. A launch with a cut tail (p.sk_tiles != 0)
// takes the instantiation built for it, which exists with two groups only. `tiles` counts (tile, split) work items;
// the grid is the smaller of that and the number of CTA pairs the device holds at once.
LaunchResult launch_gemm_pair(const LaunchEnv& env, uint32_t kind, int epi_groups, const GemmParams& p, uint64_t tiles);
// Number of CTA pairs the device can hold at once for the given variant (0 on failure).
int gemm_pair_capacity(const LaunchEnv& env, uint32_t kind, int epi_groups);

#define MMEB200_DECLARE_SINGLE(NAME) LaunchResult NAME(const LaunchEnv& env, const GemmParams& p, unsigned grid);
#define MMEB200_DECLARE_PAIR(NAME)                                                      \
    LaunchResult NAME(const LaunchEnv& env, const GemmParams& p, uint64_t tiles);        \
    int NAME##_capacity(const LaunchEnv& env);
MMEB200_DECLARE_SINGLE(launch_single_f16_n256)
MMEB200_DECLARE_SINGLE(launch_single_tf32_n256)
MMEB200_DECLARE_SINGLE(launch_single_f8_n256)
MMEB200_DECLARE_SINGLE(launch_single_f16_n128)
MMEB200_DECLARE_SINGLE(launch_single_tf32_n128)
MMEB200_DECLARE_SINGLE(launch_single_f8_n128)
MMEB200_DECLARE_PAIR(launch_pair_f16_e1)
MMEB200_DECLARE_PAIR(launch_pair_tf32_e1)
MMEB200_DECLARE_PAIR(launch_pair_f8_e1)
MMEB200_DECLARE_PAIR(launch_pair_f16_e2)
MMEB200_DECLARE_PAIR(launch_pair_tf32_e2)
MMEB200_DECLARE_PAIR(launch_pair_f8_e2)
MMEB200_DECLARE_PAIR(launch_pair_f16_e2_cut)
MMEB200_DECLARE_PAIR(launch_pair_tf32_e2_cut)
MMEB200_DECLARE_PAIR(launch_pair_f8_e2_cut)
#undef MMEB200_DECLARE_SINGLE
#undef MMEB200_DECLARE_PAIR

}  // namespace mmeb200
