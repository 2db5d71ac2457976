// Picks the kernel instantiation for a (kind, variant) pair; see gemm_launch.h.
#include "gemm_launch.h"

namespace mmeb200 {

LaunchResult launch_gemm_single(const LaunchEnv& env, uint32_t kind, int block_n, const GemmParams& p, unsigned grid) {
    if (block_n == 256)
        return kind == KIND_F16 ? launch_single_f16_n256(env, p, grid) : kind == KIND_TF32 ? launch_single_tf32_n256(env, p, grid) : launch_single_f8_n256(env, p, grid);
    return kind == KIND_F16 ? launch_single_f16_n128(env, p, grid) : kind == KIND_TF32 ? launch_single_tf32_n128(env, p, grid) : launch_single_f8_n128(env, p, grid);
}

LaunchResult launch_gemm_pair(const LaunchEnv& env, uint32_t kind, int epi_groups, const GemmParams& p, uint64_t tiles) {
    if (p.sk_tiles != 0)
        return kind == KIND_F16 ? launch_pair_f16_e2_cut(env, p, tiles) : kind == KIND_TF32 ? launch_pair_tf32_e2_cut(env, p, tiles) : launch_pair_f8_e2_cut(env, p, tiles);
    if (epi_groups == 2)
        return kind == KIND_F16 ? launch_pair_f16_e2(env, p, tiles) : kind == KIND_TF32 ? launch_pair_tf32_e2(env, p, tiles) : launch_pair_f8_e2(env, p, tiles);
    return kind == KIND_F16 ? launch_pair_f16_e1(env, p, tiles) : kind == KIND_TF32 ? launch_pair_tf32_e1(env, p, tiles) : launch_pair_f8_e1(env, p, tiles);
}

int gemm_pair_capacity(const LaunchEnv& env, uint32_t kind, int epi_groups) {
    if (epi_groups == 2)
        return kind == KIND_F16 ? launch_pair_f16_e2_capacity(env) : kind == KIND_TF32 ? launch_pair_tf32_e2_capacity(env) : launch_pair_f8_e2_capacity(env);
    return kind == KIND_F16 ? launch_pair_f16_e1_capacity(env) : kind == KIND_TF32 ? launch_pair_tf32_e1_capacity(env) : launch_pair_f8_e1_capacity(env);
}

}  // namespace mmeb200
