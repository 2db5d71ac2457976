// Persistent, warp-specialised tcgen05 GEMM for sm_100a. One kernel serves (batched) GEMM in all
// four operand orientations and, through im2col-mode TMA loads, the implicit-GEMM convolutions
// (forward, dedx and dedw). It stands in for the reference's per-element dot-product loop
// (doMatrixMultiplicationFloat / doGemmWorkerFloat, mme/mme_reference/mme_reference_impl.cpp:914-956,
// 1022-1053) and, with the fused epilogue, for the cast that doActivation performs afterwards
// (mme_reference_impl.cpp:661-689,1143-1245).
//
// CTA layout (256 threads):
//   warp 0, 3   TMA producers (A and B): fill a ring of STAGES operand tiles (A: 128 x 128 B,
//               B: BLOCK_N x 128 B, both 128-byte swizzled) and signal full[stage] through complete_tx.
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BLOCK_N, K=32 B) into one of
//               two fp32 accumulators in tensor memory; tcgen05.commit frees the stage / publishes
//               the accumulator.
//   warp 2      allocates and frees tensor memory.
//   warps 4-7   epilogue: tcgen05.ld the accumulator (lane = row), scale, optional ReLU + rounded
//               cast, then either stage 128-byte column chunks in shared memory for TMA stores
//               (aligned outputs) or store directly (unaligned outputs, split-K partials).
//               Runs concurrently with the next tile's main loop.
// Tiles are walked in a grouped raster so that concurrently resident CTAs share operand panels
// in L2. Every mbarrier wait is bounded; a wait that gives up writes a code to p.status and the
// CTA leaves through the normal teardown.
#pragma once
#include "numerics.cuh"
#include "ptx_sm100.cuh"
#include "schedule.cuh"

namespace mmeb200 {

constexpr int kRowBytes = 128;     // bytes of K per stage row = one swizzle span
constexpr int kUmmaKBytes = 32;    // bytes of K consumed by one tcgen05.mma
constexpr int kGemmThreads = 256;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

enum : uint32_t { A_TILED = 0, A_IM2COL = 1 };
enum : uint32_t { KIND_F16 = 0, KIND_TF32 = 1, KIND_F8 = 2 };
enum : uint32_t { EPI_GENERIC = 0, EPI_F32 = 1, EPI_BF16_RNE = 2, EPI_FP8_HW = 3 };
enum : uint32_t {
    WAIT_OK = 0,
    WAIT_PRODUCER_EMPTY = 1,
    WAIT_MMA_FULL = 2,
    WAIT_MMA_TMEM_EMPTY = 3,
    WAIT_EPILOGUE_TMEM_FULL = 4,
    SMEM_MISALIGNED = 5,
    WAIT_STREAMK_PARTIAL = 6,
    CUT_TAIL_WITHOUT_HELPERS = 7
};

struct ConvGeom {
    // A operand = activation tensor (C, W, H, N) read in im2col mode.
    int32_t out_w, out_h;        // number of base positions per row / column (the GEMM's pixel grid)
    int32_t stride_w, stride_h;  // traversal stride
    int32_t lower_w, lower_h;    // coordinate of base position 0
    int32_t dil_w, dil_h;
    int32_t taps_w, taps_h;      // filter extent S, R
    int32_t flip;                // 1: tap (s,r) uses offset (S-1-s, R-1-r) (dedx)
    int32_t channels;            // C of the activation tensor
    int32_t k_blocks_per_tap;    // fwd/dedx: k blocks that share a tap
    int32_t b_tap_local;         // dedx: B's K coordinate restarts per tap, B rows advance by b_tap_rows
    int32_t b_tap_rows;          // dedx: B rows from one tap of a filter row to the next (C, or a multiple for a parity class)
    int32_t b_tap_rows_r;        // dedx: B rows from one filter row to the next used one
    int32_t b_row0;              // dedx: B row of the first tap used
    int32_t pixels_along_k;      // dedw: pixels run along K, (tap, channel) along M
    // dedx of a strided convolution: one launch computes one parity class of dX positions (those a given subset of the
    // taps reaches, RefIm2Col::internalDoCol2Im, mme/mme_reference/im2col.cpp:93-132). GEMM row (n, i, j) of the class's
    // out_h x out_w grid is stored at element out_base + n * out_stride_n + i * out_stride_h + j * out_stride_w.
    int32_t out_grid;            // 0: rows are out_ld apart
    int64_t out_base, out_stride_n, out_stride_h, out_stride_w;
};

struct GemmParams {
    CUtensorMap tm_a;
    CUtensorMap tm_b;
    CUtensorMap tm_out;      // output as (N, M, b0, b1, b2), box 128 B x 32 rows (one per epilogue warp); used when tma_store != 0
    uint32_t tma_store;
    uint32_t M, N, K;
    uint32_t block_k;       // elements per k block (128 B / element size)
    uint32_t num_k_blocks;  // over the whole K
    uint32_t m_tiles, n_tiles, batches, split_k;
    uint32_t raster_gm;     // m tiles per raster group: tiles of a group run together and share B panels in L2
    uint32_t tile_n;        // CTA-pair kernel: columns of an output tile (a multiple of 32, at most 256); n_tiles counts these
    uint32_t b_cta_bytes;   // CTA-pair kernel: bytes of B one CTA stages per k block (its tile_n / 2 columns)
    uint32_t bsz[3];
    uint32_t a_bcast[3], b_bcast[3];
    uint32_t a_mn_major, b_mn_major;
    uint32_t a_mode;
    uint32_t idesc;
    uint32_t elem_bytes;
    ConvGeom conv;
    // epilogue
    void* out;               // split_k == 1: final output; else fp32 workspace [split][batch][M][N]
    uint32_t out_dtype;
    uint32_t has_cast;
    uint32_t epi_mode;       // EPI_*: which epilogue body applies (uniform per launch)
    uint64_t out_ld;         // elements between output rows
    uint64_t out_bstride[3]; // elements between batches
    float scale;
    Fp8HwCast hw;            // EPI_FP8_HW
    CastSpec cast;
    uint32_t rng_philox;
    uint64_t rng_seed, rng_offset;
    uint32_t* status;
    // Device-side predicate: when `pred` is set, the launch does its work only if (*pred != 0) == (pred_nonzero != 0) and
    // exits at once otherwise. The planner enqueues both forms of a GEMM whose choice depends on the operands' contents
    // (fp8 codes that the tensor cores would read differently) and lets the device pick, with no host round trip.
    const uint32_t* pred;
    uint32_t pred_nonzero;
    // Cut tail of the CTA-pair kernel (split_k == 1). With whole tiles only, the last `tiles % pairs` tiles make a wave that
    // leaves pairs idle. The planner cuts each of those sk_tiles tiles (the last ones of the raster order) along K into a
    // head of sk_head k blocks and sk_pieces further pieces of sk_piece k blocks. Pair t < sk_tiles computes the head of cut
    // tile t; the other pairs share the pieces, last piece first (PairSchedule); every pair then goes on to its whole tiles.
    // The sums travel down a tile's pieces: the pair with piece q waits for slot (tile, q + 1) unless q is the last piece,
    // adds it to its raw fp32 accumulator, writes the result to slot (tile, q) = tile * sk_pieces + q - 1 of sk_ws and then
    // stores sk_gen to its epilogue warps' words of sk_flags; the pair with the head waits for slot (tile, 1), adds it and
    // does the tile's epilogue. Nobody waits for a pair that itself waits for work that has not started.
    uint32_t sk_tiles;       // 0: every tile is computed whole by one pair
    uint32_t sk_head, sk_piece, sk_pieces;
    float* sk_ws;            // [slot][CTA of the pair][column 0..255][row 0..127] floats: 128 KB per CTA
    uint32_t* sk_flags;      // [slot][CTA of the pair][16]: one word per epilogue warp of the writer
    uint32_t sk_gen;         // differs from every earlier launch that used the same flags; never 0
};
constexpr uint32_t kSkSlotFloats = 8 * kBlockM * 32;   // one CTA's 128 x 256 partial accumulator
constexpr uint32_t kSkFlagsPerCta = 16;

// What the pair with the head of a cut tile adds to its accumulator before the cast: this CTA's part of the slot `ws` when
// count != 0. col0: first column of the warp's share within the tile.
struct SkFix {
    const float* ws;
    uint32_t count;
    uint32_t col0;
};
// 32 accumulator columns of this lane's row (tile column `col`, a multiple of 32) plus the slot's values for them. A slot
// holds its CTA's 128 x 256 sums column by column, so the 32 lanes of a warp (32 consecutive rows) read and write 128
// consecutive bytes per column. The loads are issued before the wait for the accumulator's own load.
__device__ __forceinline__ void tmem_ld_wait_add(uint32_t (&v)[32], const SkFix& fix, uint32_t col, uint32_t row_in_cta) {
    if (fix.count) {
        const float* src = fix.ws + uint64_t(col) * kBlockM + row_in_cta;
        float w[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = __ldcg(src + j * kBlockM);   // written by another SM during this launch: read past L1
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + w[j]);
    } else {
        tmem_ld_wait();
    }
}
// A piece of a cut tile: this warp's 32 rows x tile_cols raw accumulator columns, plus the running sum of the pieces
// after it (`above`, nullptr for the last piece), into its CTA's slot.
static __device__ __noinline__ void epilogue_partial(float* slot, const float* above, uint32_t col0, uint32_t tile_cols, uint32_t tmem_acc,
                                                     uint32_t row_in_cta) {
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < tile_cols; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_acc + c0, v);
        const uint64_t at = uint64_t(col0 + c0) * kBlockM + row_in_cta;
        if (above) {
            float w[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = __ldcg(above + at + j * kBlockM);   // in flight while the accumulator arrives
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + w[j]);
        } else {
            tmem_ld_wait();
        }
        float* dst = slot + at;
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j * kBlockM] = __uint_as_float(v[j]);
    }
}

__device__ __forceinline__ bool launch_is_predicated_off(const uint32_t* pred, uint32_t pred_nonzero) {
    return pred != nullptr && ((*pred != 0u) != (pred_nonzero != 0u));
}

template <int BLOCK_N, int STAGES>
struct GemmSmem {
    static constexpr int kABytes = kBlockM * kRowBytes;
    static constexpr int kBBytes = BLOCK_N * kRowBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 256;    // after the staging buffers, which need 1024-byte alignment
    static constexpr int kOutStageBytes = 2 * kBlockM * kRowBytes;
    // No alignment slack: the dynamic shared memory is declared 1024-byte aligned and the kernel checks it. The CTA then
    // leaves about 2.8 KB of the SM's shared memory free, enough for a small block of another kernel (the dedw exchange's
    // wait-and-add kernels) to share the SM with it.
    static constexpr int kTotal = STAGES * kStageBytes + kOutStageBytes + kBarrierBytes;
};

// One accumulator value before its cast: scale, NaN canonicalisation, optional ReLU.
__device__ __forceinline__ uint32_t epilogue_prepare(uint32_t acc, const GemmParams& p) {
    uint32_t bits = __float_as_uint(__uint_as_float(acc) * p.scale);
    if (f32_is_nan(bits)) bits = kF32CanonNan;
    if (p.cast.relu) bits = relu_bits(bits);
    return bits;
}

// bf16 output in any rounding mode, straight-line: 32 values in v become 16 packed words. Stochastic rounding draws one
// Philox block per EIGHT elements (16 random bits each, philox_halves8); the stream position of the 32 is a multiple of 8.
template <int RM>
__device__ __forceinline__ void epilogue_bf16_flat(uint32_t (&v)[32], const GemmParams& p, uint64_t flat_index) {
    const bool clip = p.cast.clip, ftz = p.cast.ftz, clip_inf_in = p.cast.clip_inf_in;
    if constexpr (RM == RM_SR) {
        if (p.rng_philox && !ftz && !p.cast.relu) {
            // the rounding as one addition per element (sr_bf16_group8); NaN needs no canonical form, every NaN gives 0x7FFF
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t c[4], x[8], w[4];
                philox_block8(p.rng_seed, p.rng_offset, flat_index + 8 * g, c);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = __float_as_uint(__uint_as_float(v[8 * g + e]) * p.scale);
                sr_bf16_group8(x, c, clip, clip_inf_in, w);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[4 * g + e] = w[e];
            }
            return;
        }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t rnd[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u}, o[8];
        if (RM == RM_SR && p.rng_philox) philox_halves8(p.rng_seed, p.rng_offset, flat_index + 8 * g, rnd);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = f32_to_bf16_flat<RM>(epilogue_prepare(v[8 * g + e], p), rnd[e], clip, ftz, clip_inf_in);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[4 * g + e] = o[2 * e] | (o[2 * e + 1] << 16);   // words 4g .. 4g+3 lie below every value still to be read
    }
}

// fp8 output without the flush flags, straight-line: 32 values in v become 8 packed words. The stochastic modes draw one
// Philox block per eight elements, as the bf16 cast does.
template <int RM>
__device__ __forceinline__ void epilogue_fp8_flat(uint32_t (&v)[32], const GemmParams& p, uint64_t flat_index) {
    const int exp_width = p.cast.exp_width, bias = p.cast.bias, mode = p.cast.mode;
    const bool clip = p.cast.clip, clip_inf_in = p.cast.clip_inf_in;
    if constexpr (RM == RM_SR) {
        if (p.rng_philox && !p.cast.relu) {
            // the rounding as one addition per element (sr_fp8_group8); the accumulator's NaN is the positive canonical one
            const Fp8SrSpec sp = fp8_sr_spec(exp_width, bias, mode);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t c[4], x[8], w[2];
                philox_block8(p.rng_seed, p.rng_offset, flat_index + 8 * g, c);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = __float_as_uint(__uint_as_float(v[8 * g + e]) * p.scale);
                sr_fp8_group8(x, c, sp, exp_width, bias, mode, clip, clip_inf_in, true, w);
                v[2 * g] = w[0];
                v[2 * g + 1] = w[1];
            }
            return;
        }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t rnd[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u}, o[8];
        if ((RM == RM_SR || RM == RM_SR_NE_DNORM) && p.rng_philox) philox_halves8(p.rng_seed, p.rng_offset, flat_index + 8 * g, rnd);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = f32_to_fp8_flat<RM>(epilogue_prepare(v[8 * g + e], p), exp_width, bias, rnd[e], mode, clip, clip_inf_in);
        v[2 * g] = o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24);        // words 2g, 2g+1 lie below every value still to be read
        v[2 * g + 1] = o[4] | (o[5] << 8) | (o[6] << 16) | (o[7] << 24);
    }
}

// The general cast, every flag and every input: a few hundred instructions per element with data-dependent branches.
// It runs as a rolled loop over groups of four elements of an array that the loop may index, which keeps the code small.
__device__ __forceinline__ void epilogue_general(uint32_t (&t)[32], const GemmParams& p, uint32_t out_elem, uint64_t flat_index) {
    const bool philox = p.rng_philox != 0, aligned = ((p.rng_offset + flat_index) & 3u) == 0;
#pragma unroll 1
    for (int q = 0; q < 8; ++q) {
        uint32_t rnd[4] = {0u, 0u, 0u, 0u};
        if (philox) {
            if (aligned) {
                philox_halves4(p.rng_seed, p.rng_offset, flat_index + 4 * q, rnd);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) rnd[e] = cast_random_word(p.rng_seed, p.rng_offset, flat_index + 4 * q + e);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) t[4 * q + e] = cast_from_f32(epilogue_prepare(t[4 * q + e], p), p.cast, rnd[e]);
    }
    if (out_elem == 2) {
#pragma unroll 1
        for (int j = 0; j < 16; ++j) t[j] = (t[2 * j] & 0xFFFFu) | (t[2 * j + 1] << 16);
    } else if (out_elem == 1) {
#pragma unroll 1
        for (int j = 0; j < 8; ++j)
            t[j] = (t[4 * j] & 0xFFu) | ((t[4 * j + 1] & 0xFFu) << 8) | ((t[4 * j + 2] & 0xFFu) << 16) | (t[4 * j + 3] << 24);
    }
}

// Every cast that is not one of the inlined paths: the straight-line fp8 casts where they apply (one Philox block per
// four elements needs the stream position aligned), else the general cast. One out-of-line copy serves every kernel and
// both store paths; its argument lives in local memory, so the caller hands it a copy of the accumulator registers
// (an array whose address is taken is in memory everywhere, the fast paths included).
static __device__ __noinline__ void epilogue_cast_any(uint32_t (&v)[32], const GemmParams& p, uint32_t out_elem, uint64_t flat_index) {
    const bool stream_ok = !p.rng_philox || ((p.rng_offset + flat_index) & 7u) == 0;
    if (stream_ok && dtype_is_fp8(p.cast.out_dtype) && !p.cast.ftz && !p.cast.sftz) {
        switch (p.cast.rm) {
            case RM_UP: epilogue_fp8_flat<RM_UP>(v, p, flat_index); return;
            case RM_DOWN: epilogue_fp8_flat<RM_DOWN>(v, p, flat_index); return;
            case RM_HAZ: epilogue_fp8_flat<RM_HAZ>(v, p, flat_index); return;
            default: break;   // the inlined modes arrive here only with an unaligned random stream
        }
    }
    epilogue_general(v, p, out_elem, flat_index);
}

// Turns 32 fp32 accumulator columns into 32 outputs of the launch's output type, packed little-endian
// into the first 8 * out_elem words of v: scale, NaN canonicalisation, optional ReLU, rounded cast.
__device__ __forceinline__ void epilogue_convert(uint32_t (&v)[32], const GemmParams& p, uint32_t out_elem, uint64_t flat_index) {
    if (p.epi_mode == EPI_BF16_RNE) {
        // round-to-nearest-even with no flags: the hardware conversion gives the reference's bits
        // (NaN -> 0x7FFF, denormals kept)
        if (p.scale == 1.0f) {   // operands with the tensor cores' own exponent bias: nothing to fold
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                uint32_t packed;
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(__uint_as_float(v[2 * j + 1])), "f"(__uint_as_float(v[2 * j])));
                v[j] = packed;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float lo = __uint_as_float(v[2 * j]) * p.scale, hi = __uint_as_float(v[2 * j + 1]) * p.scale;
                uint32_t packed;
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
                v[j] = packed;
            }
        }
    } else if (p.epi_mode == EPI_F32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const uint32_t bits = __float_as_uint(__uint_as_float(v[j]) * p.scale);
            v[j] = f32_is_nan(bits) ? kF32CanonNan : bits;
        }
    } else if (p.epi_mode == EPI_FP8_HW) {
        // hardware conversion after an exact rescale (f32x4_to_fp8_hw)
        const bool relu = p.cast.relu != 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            float x[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                x[e] = __uint_as_float(v[4 * q + e]) * p.scale;
                if (relu) x[e] = x[e] > 0.0f ? x[e] : 0.0f;          // NaN and -0 become +0, as std::max(0.f, x)
            }
            v[q] = f32x4_to_fp8_hw(x, p.hw, true);   // the accumulator's NaN is canonical (positive); word q lies below every value still to be read
        }
    } else {
        // bf16 in the other rounding modes: some twenty instructions per element, inlined on the accumulator registers
        if (p.cast.out_dtype == DT_BF16 && (!p.rng_philox || ((p.rng_offset + flat_index) & 7u) == 0)) {
            switch (p.cast.rm) {
                case RM_NE: epilogue_bf16_flat<RM_NE>(v, p, flat_index); break;
                case RM_UP: epilogue_bf16_flat<RM_UP>(v, p, flat_index); break;
                case RM_DOWN: epilogue_bf16_flat<RM_DOWN>(v, p, flat_index); break;
                case RM_SR: epilogue_bf16_flat<RM_SR>(v, p, flat_index); break;
                case RM_HAZ: epilogue_bf16_flat<RM_HAZ>(v, p, flat_index); break;
                default: epilogue_bf16_flat<RM_Z>(v, p, flat_index); break;   // every other mode truncates
            }
            return;
        }
        // fp8 in the common rounding modes, inlined as well (out of line, through local memory, stochastic rounding
        // measured 0.67 ms on 8192^3 against 0.40 ms inlined); the rarer modes stay out of line to bound the build time
        if (dtype_is_fp8(p.cast.out_dtype) && !p.cast.ftz && !p.cast.sftz && (!p.rng_philox || ((p.rng_offset + flat_index) & 7u) == 0)) {
            switch (p.cast.rm) {
                case RM_NE: epilogue_fp8_flat<RM_NE>(v, p, flat_index); return;
                case RM_Z: epilogue_fp8_flat<RM_Z>(v, p, flat_index); return;
                case RM_SR: epilogue_fp8_flat<RM_SR>(v, p, flat_index); return;
                case RM_SR_NE_DNORM: epilogue_fp8_flat<RM_SR_NE_DNORM>(v, p, flat_index); return;
                default: break;
            }
        }
        uint32_t t[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) t[j] = v[j];
        epilogue_cast_any(t, p, out_elem, flat_index);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = t[j];     // at most 16 packed words (the fp32 cast with flags: all 32)
        if (out_elem == 4) {
#pragma unroll
            for (int j = 16; j < 32; ++j) v[j] = t[j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Operand feeds: the coordinate bookkeeping of the two TMA producer threads, shared by the
// single-CTA and the CTA-pair kernel (PAIR selects the load form whose completion may be signalled
// on the partner CTA's barrier). Everything that is constant inside a tile is computed in
// begin_tile; coordinates then advance incrementally, with no division per k block.
// ---------------------------------------------------------------------------------------------
template <bool PAIR>
__device__ __forceinline__ void feed_load_tiled(void* dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
    if constexpr (PAIR) tma_load_5d_pair(dst, m, bar, c0, c1, c2, c3, c4);
    else tma_load_5d(dst, m, bar, c0, c1, c2, c3, c4);
}
template <bool PAIR>
__device__ __forceinline__ void feed_load_im2col(void* dst, const CUtensorMap* m, uint32_t bar, int c, int w, int h, int n, uint16_t ow,
                                                 uint16_t oh) {
    if constexpr (PAIR) tma_load_im2col_4d_pair(dst, m, bar, c, w, h, n, ow, oh);
    else tma_load_im2col_4d(dst, m, bar, c, w, h, n, ow, oh);
}

// A operand: 128 rows (or, MN-major, 128 columns of the stored matrix) starting at m0.
struct AFeed {
    bool a_mn, im2col, pix_k;
    uint32_t a_groups, mn_group_elems, mn_group_bytes, block_k;
    uint32_t m0;
    int ab0, ab1, ab2;
    uint32_t k_elem;                           // K coordinate of a plain (tiled) operand
    int pw, ph, pn;                            // fwd / dedx: base position of the tile's first pixel
    uint32_t tap_s, tap_r, k_in_tap;           // fwd / dedx: filter tap and channel offset
    uint32_t pq, pp, pimg;                     // dedw: pixel position of the k block
    uint16_t g_off_w[4], g_off_h[4];
    int g_c[4];

    __device__ __forceinline__ void setup(const GemmParams& p) {
        a_mn = p.a_mn_major != 0;
        im2col = p.a_mode == A_IM2COL;
        pix_k = im2col && p.conv.pixels_along_k;
        a_groups = a_mn ? (kBlockM * p.elem_bytes) / kRowBytes : 1;   // <= 4
        mn_group_elems = kRowBytes / p.elem_bytes;
        mn_group_bytes = p.block_k * kRowBytes;
        block_k = p.block_k;
    }
    __device__ __forceinline__ void begin_tile(const GemmParams& p, uint32_t first_row, uint32_t batch, uint32_t kb_begin) {
        m0 = first_row;
        uint32_t b = batch;
        const uint32_t i0 = b % p.bsz[0]; b /= p.bsz[0];
        const uint32_t i1 = b % p.bsz[1]; b /= p.bsz[1];
        ab0 = p.a_bcast[0] ? 0 : int(i0);
        ab1 = p.a_bcast[1] ? 0 : int(i1);
        ab2 = p.a_bcast[2] ? 0 : int(b);
        k_elem = kb_begin * block_k;
        pw = ph = pn = 0;
        tap_s = tap_r = k_in_tap = 0;
        pq = pp = pimg = 0;
#pragma unroll
        for (int g = 0; g < 4; ++g) { g_off_w[g] = 0; g_off_h[g] = 0; g_c[g] = 0; }
        if (im2col && !pix_k) {
            const uint32_t q = m0 % p.conv.out_w;
            const uint32_t rest = m0 / p.conv.out_w;
            pw = int(q) * p.conv.stride_w + p.conv.lower_w;
            ph = int(rest % p.conv.out_h) * p.conv.stride_h + p.conv.lower_h;
            pn = int(rest / p.conv.out_h);
            const uint32_t tap = kb_begin / p.conv.k_blocks_per_tap;
            k_in_tap = (kb_begin % p.conv.k_blocks_per_tap) * block_k;
            tap_s = tap % p.conv.taps_w;
            tap_r = tap / p.conv.taps_w;
        } else if (pix_k) {
            const uint32_t pix = kb_begin * block_k;
            pq = pix % p.conv.out_w;
            const uint32_t rest = pix / p.conv.out_w;
            pp = rest % p.conv.out_h;
            pimg = rest / p.conv.out_h;
#pragma unroll
            for (uint32_t g = 0; g < 4; ++g) {
                if (g < a_groups) {
                    const uint32_t m = m0 + g * mn_group_elems;
                    const uint32_t tp = m / p.conv.channels;
                    g_c[g] = int(m % p.conv.channels);
                    g_off_w[g] = uint16_t((tp % p.conv.taps_w) * p.conv.dil_w);
                    g_off_h[g] = uint16_t((tp / p.conv.taps_w) * p.conv.dil_h);
                }
            }
        }
    }
    // issues the loads of one k block into a_dst, completion on `bar`, and steps to the next k block
    template <bool PAIR>
    __device__ __forceinline__ void load(const GemmParams& p, uint8_t* a_dst, uint32_t bar) {
        if (!im2col) {
            if (!a_mn) {
                feed_load_tiled<PAIR>(a_dst, &p.tm_a, bar, int(k_elem), int(m0), ab0, ab1, ab2);
            } else {
#pragma unroll
                for (uint32_t g = 0; g < 4; ++g)
                    if (g < a_groups) feed_load_tiled<PAIR>(a_dst + g * mn_group_bytes, &p.tm_a, bar, int(m0 + g * mn_group_elems), int(k_elem), ab0, ab1, ab2);
            }
            k_elem += block_k;
        } else if (!pix_k) {
            const uint32_t s = p.conv.flip ? p.conv.taps_w - 1 - tap_s : tap_s;
            const uint32_t r = p.conv.flip ? p.conv.taps_h - 1 - tap_r : tap_r;
            feed_load_im2col<PAIR>(a_dst, &p.tm_a, bar, int(k_in_tap), pw, ph, pn, uint16_t(s * p.conv.dil_w), uint16_t(r * p.conv.dil_h));
            k_in_tap += block_k;
            if (k_in_tap >= uint32_t(p.conv.k_blocks_per_tap) * block_k) {
                k_in_tap = 0;
                if (++tap_s == uint32_t(p.conv.taps_w)) { tap_s = 0; ++tap_r; }
            }
        } else {
            const int w0 = int(pq) * p.conv.stride_w + p.conv.lower_w;
            const int h0 = int(pp) * p.conv.stride_h + p.conv.lower_h;
#pragma unroll
            for (uint32_t g = 0; g < 4; ++g)
                if (g < a_groups) feed_load_im2col<PAIR>(a_dst + g * mn_group_bytes, &p.tm_a, bar, g_c[g], w0, h0, int(pimg), g_off_w[g], g_off_h[g]);
            pq += block_k;
            while (pq >= uint32_t(p.conv.out_w)) {
                pq -= p.conv.out_w;
                if (++pp == uint32_t(p.conv.out_h)) { pp = 0; ++pimg; }
            }
        }
    }
};

// B operand: COLS columns of the output (rows of the stored K-major matrix) starting at n_first.
template <int COLS>
struct BFeed {
    bool b_mn, tap_local;
    uint32_t b_groups, mn_group_elems, mn_group_bytes, block_k;
    uint32_t n_first, row, k_elem, k_wrap, tap_s;
    int bb0, bb1, bb2;

    // cols: columns this CTA stages (COLS, or fewer in the CTA-pair kernel when the planner narrows the tile)
    __device__ __forceinline__ void setup(const GemmParams& p, uint32_t cols = COLS) {
        b_mn = p.b_mn_major != 0;
        tap_local = p.conv.b_tap_local != 0;
        b_groups = b_mn ? (cols * p.elem_bytes + kRowBytes - 1) / kRowBytes : 1;   // <= 8
        mn_group_elems = kRowBytes / p.elem_bytes;
        mn_group_bytes = p.block_k * kRowBytes;
        block_k = p.block_k;
    }
    __device__ __forceinline__ void begin_tile(const GemmParams& p, uint32_t first_col, uint32_t batch, uint32_t kb_begin) {
        n_first = first_col;
        uint32_t b = batch;
        const uint32_t i0 = b % p.bsz[0]; b /= p.bsz[0];
        const uint32_t i1 = b % p.bsz[1]; b /= p.bsz[1];
        bb0 = p.b_bcast[0] ? 0 : int(i0);
        bb1 = p.b_bcast[1] ? 0 : int(i1);
        bb2 = p.b_bcast[2] ? 0 : int(b);
        k_elem = kb_begin * block_k;
        row = n_first;
        tap_s = 0;
        if (tap_local) {  // dedx: B's K coordinate restarts at every filter tap, its rows move on to the next tap's
            const uint32_t tap = kb_begin / p.conv.k_blocks_per_tap;
            k_elem = (kb_begin % p.conv.k_blocks_per_tap) * block_k;
            tap_s = tap % uint32_t(p.conv.taps_w);
            row = n_first + uint32_t(p.conv.b_row0) + tap_s * uint32_t(p.conv.b_tap_rows) + (tap / uint32_t(p.conv.taps_w)) * uint32_t(p.conv.b_tap_rows_r);
        }
        k_wrap = tap_local ? uint32_t(p.conv.k_blocks_per_tap) * block_k : 0xFFFFFFFFu;
    }
    template <bool PAIR>
    __device__ __forceinline__ void load(const GemmParams& p, uint8_t* b_dst, uint32_t bar) {
        if (!b_mn) {
            feed_load_tiled<PAIR>(b_dst, &p.tm_b, bar, int(k_elem), int(row), bb0, bb1, bb2);
        } else {
#pragma unroll
            for (uint32_t g = 0; g < 8; ++g)
                if (g < b_groups) feed_load_tiled<PAIR>(b_dst + g * mn_group_bytes, &p.tm_b, bar, int(n_first + g * mn_group_elems), int(k_elem), bb0, bb1, bb2);
        }
        k_elem += block_k;
        if (k_elem >= k_wrap) {
            k_elem = 0;
            row += p.conv.b_tap_rows;
            if (++tap_s == uint32_t(p.conv.taps_w)) { tap_s = 0; row += p.conv.b_tap_rows_r - p.conv.taps_w * p.conv.b_tap_rows; }
        }
    }
};

// Stores 32 consecutive outputs of one row (v[0 .. 8 * elem) holds them packed) straight to global memory: 16-byte
// stores when the 32 are all inside the matrix and the address allows, element stores on ragged edges.
__device__ __forceinline__ void store_row32(const uint32_t (&v)[32], uint8_t* dst, uint32_t elem, uint32_t ncols) {
    if (ncols == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
        if (elem == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else if (elem == 2) {
#pragma unroll
            for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    } else {
        // ragged edge or unaligned row: element-wise, statically indexed
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (uint32_t(j) < ncols) {
                if (elem == 4) reinterpret_cast<uint32_t*>(dst)[j] = v[j];
                else if (elem == 2) reinterpret_cast<uint16_t*>(dst)[j] = uint16_t(v[j / 2] >> (16 * (j & 1)));
                else dst[j] = uint8_t(v[j / 4] >> (8 * (j & 3)));
            }
        }
    }
}

// Epilogue of one output tile, run by one epilogue warp for its 32 rows: reads `tile_cols` accumulator columns (a
// multiple of 32) from tensor memory (tmem_acc = the warp's lane window of the tile's accumulator), converts and stores
// them. m0 is the first row of the CTA's 128-row block, n0 the first column.
template <bool FIX = false>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, uint32_t tile_cols, uint32_t m0, uint32_t n0, uint32_t batch, uint32_t split,
                                              uint32_t tmem_acc, uint8_t* stage_out, uint32_t& store_buf, uint32_t sub, uint32_t lane,
                                              uint32_t out_elem, const SkFix& fix = SkFix{nullptr, 0u, 0u}) {
    const uint32_t row = m0 + sub * 32 + lane;
    uint32_t bi[3];
    {
        uint32_t b = batch;
        bi[0] = b % p.bsz[0]; b /= p.bsz[0];
        bi[1] = b % p.bsz[1]; b /= p.bsz[1];
        bi[2] = b;
    }
    uint64_t flat_row = (uint64_t(batch) * p.M + row) * p.N;  // index base for the random stream
    uint64_t base_off;
    if (p.split_k > 1) {
        base_off = (uint64_t(split) * p.batches + batch) * uint64_t(p.M) * p.N + uint64_t(row) * p.N;
    } else if (p.conv.out_grid) {
        // a parity class of dX: the row is pixel (n, i, j) of the class's grid; the tensor is dense, so the element offset
        // is also the output's flat index (the random stream's position)
        const uint32_t j = row % uint32_t(p.conv.out_w), t = row / uint32_t(p.conv.out_w);
        const uint32_t i = t % uint32_t(p.conv.out_h), n = t / uint32_t(p.conv.out_h);
        base_off = uint64_t(p.conv.out_base + int64_t(n) * p.conv.out_stride_n + int64_t(i) * p.conv.out_stride_h + int64_t(j) * p.conv.out_stride_w);
        flat_row = base_off;
    } else {
        base_off = bi[0] * p.out_bstride[0] + bi[1] * p.out_bstride[1] + bi[2] * p.out_bstride[2] + uint64_t(row) * p.out_ld;
    }
    uint32_t done_cols = 0;   // columns of the tile already stored
    if (p.tma_store) {
        // ---- stage 128-byte-wide column chunks in shared memory (128-byte swizzle) and let the
        //      copy engine write them: full-line, coalesced stores, edges clipped by the tensor map.
        //      Only whole chunks go this way: the columns after a narrowed tile's end belong to the next tile.
        const uint32_t cols_per_chunk = kRowBytes / out_elem;    // 32 fp32 / 64 bf16 / 128 fp8 columns
        const uint32_t lds_per_chunk = cols_per_chunk / 32;
        // each warp owns two 32-row x 128-byte buffers and issues its own stores: warps never
        // wait for one another here
        uint8_t* my_bufs = stage_out + sub * (2 * 32 * kRowBytes);
        const uint32_t sw = (lane & 7);
#pragma unroll 1
        for (uint32_t ch = 0; ch < tile_cols / cols_per_chunk; ++ch) {
            const uint32_t col0 = n0 + ch * cols_per_chunk;
            done_cols = (ch + 1) * cols_per_chunk;
            if (col0 >= p.N) break;  // uniform over the CTA
            uint8_t* buf = my_bufs + store_buf * (32 * kRowBytes);
            if (lane == 0) tma_store_wait_read<1>();   // the store issued two chunks ago has drained this buffer
            __syncwarp();
            uint8_t* my_row = buf + lane * kRowBytes;
#pragma unroll 1
            for (uint32_t l = 0; l < lds_per_chunk; ++l) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_acc + ch * cols_per_chunk + l * 32, v);
                if constexpr (FIX) tmem_ld_wait_add(v, fix, fix.col0 + ch * cols_per_chunk + l * 32, sub * 32 + lane);
                else tmem_ld_wait();
                epilogue_convert(v, p, out_elem, flat_row + col0 + l * 32);
                if (out_elem == 4) {
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q)
                        *reinterpret_cast<uint4*>(my_row + (((l * 8 + q) ^ sw) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else if (out_elem == 2) {
#pragma unroll
                    for (uint32_t q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4*>(my_row + (((l * 4 + q) ^ sw) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else {
#pragma unroll
                    for (uint32_t q = 0; q < 2; ++q)
                        *reinterpret_cast<uint4*>(my_row + (((l * 2 + q) ^ sw) << 4)) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_5d(&p.tm_out, buf, int(col0), int(m0 + sub * 32), int(bi[0]), int(bi[1]), int(bi[2]));
                tma_store_commit();
            }
            store_buf ^= 1;
        }
    }
    // ---- direct stores: everything when no tensor map applies (unaligned outputs, split-K partials), else the
    //      columns left over after the last whole 128-byte chunk of a narrowed tile
#pragma unroll 1
    for (uint32_t c0 = done_cols; c0 < tile_cols; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_acc + c0, v);
        if constexpr (FIX) tmem_ld_wait_add(v, fix, fix.col0 + c0, sub * 32 + lane);
        else tmem_ld_wait();
        const uint32_t col0 = n0 + c0;
        if (row >= p.M || col0 >= p.N) continue;
        const uint32_t ncols = min(32u, p.N - col0);
        uint32_t elem = 4;
        uint8_t* dst;
        if (p.split_k > 1) {
            dst = reinterpret_cast<uint8_t*>(reinterpret_cast<float*>(p.out) + base_off + col0);
        } else {
            elem = out_elem;
            dst = reinterpret_cast<uint8_t*>(p.out) + (base_off + col0) * out_elem;
            epilogue_convert(v, p, out_elem, flat_row + col0);
        }
        store_row32(v, dst, elem, ncols);   // v[0 .. 8*elem) holds 32 packed outputs
    }
}

template <int KIND, int BLOCK_N, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
    using S = GemmSmem<BLOCK_N, STAGES>;
    if (p.pred) griddep_wait();   // the predicate word comes from an earlier kernel of the stream
    if (launch_is_predicated_off(p.pred, p.pred_nonzero)) return;   // uniform over the grid, before anything is set up
    griddep_launch_dependents();   // the next kernel of the stream may become resident as this grid's CTAs finish
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (smem_u32(smem) & 1023u) {   // the operand stages and the staging buffers need 1024-byte alignment (128-byte swizzle)
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, SMEM_MISALIGNED);
        return;
    }
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes + S::kOutStageBytes);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t total_tiles = p.m_tiles * p.n_tiles * p.batches * p.split_k;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 2);   // the A producer and the B producer each arrive once
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full_bar[b], 1);
            mbar_init(&tmem_empty_bar[b], 128);
        }
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_a);
        tma_prefetch_desc(&p.tm_b);
        if (p.tma_store) tma_prefetch_desc(&p.tm_out);
    }
    if (warp == 2) {
        tmem_alloc(tmem_holder, 2 * BLOCK_N);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    griddep_wait();   // set-up touched no global memory; what follows may depend on the kernel before this one

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer for A
        // One thread feeds A's half of the ring (warp 3 feeds B's). Everything that does not
        // change inside a tile is computed before the k loop, and coordinates advance
        // incrementally: no division per k block.
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            AFeed feed;
            feed.setup(p);
            for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                feed.begin_tile(p, tc.m0, tc.batch, tc.kb_begin);
                for (uint32_t kb = tc.kb_begin; kb < tc.kb_end; ++kb) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, kWaitLimitNs)) {
                        atomicCAS(p.status, 0u, WAIT_PRODUCER_EMPTY);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_bar[stage], S::kABytes);
                    feed.load<false>(p, smem + stage * S::kStageBytes, smem_u32(&full_bar[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ------------------------------------------------------------------ TMA producer for B
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            BFeed<BLOCK_N> feed;
            feed.setup(p);
            for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                feed.begin_tile(p, tc.n0 * BLOCK_N, tc.batch, tc.kb_begin);
                for (uint32_t kb = tc.kb_begin; kb < tc.kb_end; ++kb) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, kWaitLimitNs)) {
                        atomicCAS(p.status, 0u, WAIT_PRODUCER_EMPTY);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full_bar[stage], S::kBBytes);
                    feed.load<false>(p, smem + stage * S::kStageBytes + S::kABytes, smem_u32(&full_bar[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // One thread issues all MMAs. The two shared-memory descriptors of a stage differ from
        // stage 0's only in the start-address field, so each MMA costs two 64-bit adds.
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t mn_k_step = (kUmmaKBytes / p.elem_bytes) * kRowBytes;  // MN-major: bytes per MMA along K
            const uint32_t mn_lbo = p.block_k * kRowBytes;
            const uint32_t smem_base = smem_u32(smem);
            const uint64_t a_desc0 = p.a_mn_major ? make_smem_desc(smem_base, mn_lbo, 1024) : make_smem_desc(smem_base, 16, 1024);
            const uint64_t b_desc0 = p.b_mn_major ? make_smem_desc(smem_base + S::kABytes, mn_lbo, 1024)
                                                  : make_smem_desc(smem_base + S::kABytes, 16, 1024);
            const uint64_t a_step = (p.a_mn_major ? mn_k_step : uint32_t(kUmmaKBytes)) >> 4;
            const uint64_t b_step = (p.b_mn_major ? mn_k_step : uint32_t(kUmmaKBytes)) >> 4;
            constexpr uint64_t kStageUnits = S::kStageBytes >> 4;
            const uint32_t idesc = p.idesc;
            for (uint32_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                if (!mbar_wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1, kWaitLimitNs)) {
                    atomicCAS(p.status, 0u, WAIT_MMA_TMEM_EMPTY);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
                uint32_t accumulate = 0;
                for (uint32_t kb = tc.kb_begin; kb < tc.kb_end; ++kb) {
                    if (!mbar_wait_bounded(&full_bar[stage], phase, kWaitLimitNs)) {
                        atomicCAS(p.status, 0u, WAIT_MMA_FULL);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint64_t a_desc = a_desc0 + stage * kStageUnits;
                    const uint64_t b_desc = b_desc0 + stage * kStageUnits;
#pragma unroll
                    for (uint32_t k = 0; k < kRowBytes / kUmmaKBytes; ++k) {
                        umma_ss<KIND>(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc, accumulate);
                        accumulate = 1;
                    }
                    umma_commit(&empty_bar[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&tmem_full_bar[acc]);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue
        const uint32_t sub = warp & 3;  // tensor-memory sub-partition this warp may read
        uint32_t acc = 0, acc_phase = 0;
        const uint32_t out_elem = dtype_size(int(p.out_dtype));
        uint8_t* stage_out = smem + STAGES * S::kStageBytes;  // 2 x [128 rows x 128 B], 1024-aligned
        uint32_t store_buf = 0;
        for (uint32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
            const TileCoord tc = decode_tile(p, t);
            const uint32_t n0 = tc.n0 * BLOCK_N;
            bool ready = mbar_wait_bounded(&tmem_full_bar[acc], acc_phase, kWaitLimitNs);
            ready = __all_sync(0xffffffffu, ready);
            if (!ready) {
                atomicCAS(p.status, 0u, WAIT_EPILOGUE_TMEM_FULL);
                break;
            }
            tc_fence_after_sync();
            const uint32_t tmem_acc = tmem_base + acc * BLOCK_N + ((sub * 32) << 16);
            epilogue_tile(p, BLOCK_N, tc.m0, n0, tc.batch, tc.split, tmem_acc, stage_out, store_buf, sub, lane, out_elem);
            tc_fence_before_sync();
            mbar_arrive(&tmem_empty_bar[acc]);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (p.tma_store && lane == 0) tma_store_wait_all<0>();  // shared memory must outlive the copies that read it
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * BLOCK_N);
    }
}

}  // namespace mmeb200
