/*
 * mme_b200.h -- C ABI of the B200 (sm_100a) backend for the Gaudi MME compute reference.
 *
 * The reference's CPUCalculator (mme/mme_reference/mme_reference.h:108-191) keeps its C++
 * signature; its private implementation (CPUCalculatorImpl, mme/mme_reference/mme_reference_impl.cpp)
 * is the piece this library replaces. Every entry point below names the reference member it
 * stands in for. All structs are plain data, all pointers are raw, no C++ or torch type crosses
 * this boundary.
 *
 * Conventions shared with the reference:
 *   - tensors have up to 5 dims, sizes[0] is the fastest (sim_tensor_base.h:52-54), strides are
 *     in elements and strides[0] == 1;
 *   - dtype / op / rounding / inf-nan values are the numeric values of the reference enums
 *     (mme/include/mme_common/mme_common_enum.h:32-102,191-197,321-342);
 *   - conv activations are [C,W,H,(D),B], weights are [K,C,S,R,(Q)], outputs [K,Wo,Ho,(Do),B]
 *     (mme/include/general_utils.h:19-41).
 *
 * There is no CPU fallback: a call that cannot run on the GPU returns MMEB200_ERR_UNSUPPORTED
 * or MMEB200_ERR_NO_DEVICE and leaves the output untouched.
 */
#ifndef MME_B200_H
#define MME_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MMEB200_MAX_DIMS 5
#define MMEB200_MAX_CONV_DIMS 4

/* ---- status codes (the C++ shim turns any non-zero status into MME_ASSERT(0, last_error),
 *      mme/include/mme_assert.h:27-60) ---- */
enum {
    MMEB200_OK = 0,
    MMEB200_ERR_INVALID_ARG = -1,
    MMEB200_ERR_UNSUPPORTED = -2,
    MMEB200_ERR_CUDA = -3,
    MMEB200_ERR_TIMEOUT = -4,
    MMEB200_ERR_NO_DEVICE = -5,
    MMEB200_ERR_DEVICE_WAIT = -6 /* a bounded in-kernel wait gave up; context stays usable */
};

/* ---- EMmeDataType values (mme_common_enum.h:32-62) accepted by this backend ---- */
enum {
    MMEB200_FP8_143 = 9,
    MMEB200_FP8_152 = 10,
    MMEB200_BF16 = 12,
    MMEB200_FP32 = 13,
    MMEB200_FP32_IEEE = 14,
    MMEB200_TF32 = 15
};

/* ---- EMmeOpType values (mme_common_enum.h:83-102) ---- */
enum {
    MMEB200_OP_FWD = 0,
    MMEB200_OP_DEDX = 1,
    MMEB200_OP_DEDW = 2,
    MMEB200_OP_DETERMINISTIC_DEDW = 3,
    MMEB200_OP_TRANSPOSED_DEDX = 4,
    MMEB200_OP_AB = 5,
    MMEB200_OP_ABT = 6,
    MMEB200_OP_ATB = 7,
    MMEB200_OP_ATBT = 8,
    MMEB200_OP_GEMM_TRANSPOSE = 9, /* the calculator treats it as TRANS (mme_reference_impl.cpp:430-443) */
    MMEB200_OP_MEMCPY = 10,
    MMEB200_OP_TRANS = 11
};

/* ---- RoundingMode values (mme_common_enum.h:67-81) ---- */
enum {
    MMEB200_RM_NEAREST_EVEN = 0,
    MMEB200_RM_TO_ZERO = 1,
    MMEB200_RM_UP = 2,
    MMEB200_RM_DOWN = 3,
    MMEB200_RM_STOCHASTIC = 4,
    MMEB200_RM_HALF_AWAY = 6,
    MMEB200_RM_STOCHASTIC_RNE_DENORM = 7
};

/* ---- InfNanMode values (mme_common_enum.h:191-197) ---- */
enum { MMEB200_INFNAN_FULL = 0, MMEB200_INFNAN_NONE = 1, MMEB200_INFNAN_MINIMAL = 2 };

/* ---- EMmeReductionOp values (mme_common_enum.h:321-332) ---- */
enum {
    MMEB200_RED_ADD = 0,
    MMEB200_RED_SUB = 1,
    MMEB200_RED_MIN = 2,
    MMEB200_RED_MAX = 3,
    MMEB200_RED_MAX_0 = 4,
    MMEB200_RED_NONE = 5
};

/* ---- ChipType values (mme_common_enum.h:25-30). The chip selects the reference's
 *      accumulation model; this backend accumulates in fp32 on the tensor cores for all three
 *      and accepts the value only so that callers need not change. ---- */
enum { MMEB200_CHIP_GAUDI = 0, MMEB200_CHIP_GAUDI2 = 1, MMEB200_CHIP_GAUDI3 = 2 };

/* where a tensor's bytes live */
enum { MMEB200_MEM_HOST = 0, MMEB200_MEM_DEVICE = 1 };

/* source of the random word used by the stochastic rounding modes */
enum {
    MMEB200_RNG_LFSR = 0,   /* the reference's per-lane Galois LFSRs: bit-exact, standalone cast only */
    MMEB200_RNG_PHILOX = 1  /* counter-based Philox4x32-10 keyed by (seed, element position), the same stream whether the
                               cast is fused into a GEMM / convolution or runs alone. Position pos = rng_offset + flat
                               element index; the element draws 16 random bits: half (pos & 1) of word ((pos >> 1) & 3)
                               of block (pos >> 3) (third counter word 1), used as (h << 16) | 0x8000 against the
                               left-aligned discarded bits. One block serves eight elements. bf16: P(round up) is exactly
                               the discarded fraction; fp8: that fraction rounded to 16 bits */
};

/* Tensor descriptor: the plain-data image of MmeSimTensor (sim_tensor.h:9-52,
 * sim_tensor_base.h:48-158). */
typedef struct mmeb200_tensor {
    int32_t dtype;                      /* EMmeDataType value */
    int32_t dims;                       /* 1..5 */
    uint32_t sizes[MMEB200_MAX_DIMS];   /* sizes[0] fastest; unused dims = 1 */
    uint32_t strides[MMEB200_MAX_DIMS]; /* in elements; strides[0] == 1 */
    uint32_t fp_bias;                   /* fp8 exponent bias (143: 3,7,11,15; 152: 1..30) */
    int32_t inf_nan_mode;               /* InfNanMode value */
    int32_t mem_space;                  /* MMEB200_MEM_HOST or MMEB200_MEM_DEVICE */
    int32_t reserved;
    void* data;
} mmeb200_tensor;

/* ConvolutionParams (convolution_params.h:7-29). Index 0 is the W axis, 1 = H, 2 = D. */
typedef struct mmeb200_conv_params {
    int32_t dim;
    int32_t padding[MMEB200_MAX_CONV_DIMS];
    int32_t stride[MMEB200_MAX_CONV_DIMS];
    int32_t dilation[MMEB200_MAX_CONV_DIMS];
    uint32_t padding_value; /* ignored for float dtypes: the reference forces 0 (mme_reference_impl.cpp:810-824) */
    int32_t relu;
} mmeb200_conv_params;

/* The arguments of doActivation (mme_reference.h:162-172) that steer the fp32 -> out dtype cast. */
typedef struct mmeb200_cast_params {
    int32_t rounding;           /* RoundingMode value */
    int32_t relu;
    int32_t clip_fp;
    int32_t clip_inf_in;
    int32_t flush_denorms;
    int32_t stochastic_ftz_fp8;
    int32_t rng_kind;           /* MMEB200_RNG_* (used only by the stochastic modes) */
    int32_t reserved;
    uint64_t rng_seed;          /* Philox key */
    uint64_t rng_offset;        /* Philox counter base: element i uses counter rng_offset + i */
} mmeb200_cast_params;

typedef struct mmeb200_ctx mmeb200_ctx;

/* Replaces CPUCalculator::CPUCalculator (mme_reference_impl.cpp:129-200). `device` is a CUDA
 * ordinal. seed / lfsr / polynomial have the reference's meaning: lfsr == NULL gives registers
 * i+2, polynomial == 0 draws one in [25,63] from mt19937(seed). */
int mmeb200_create(mmeb200_ctx** out_ctx, int chip, int device, unsigned seed,
                   uint32_t lfsr_num_regs, const uint32_t* lfsr, uint32_t polynomial);
void mmeb200_destroy(mmeb200_ctx* ctx);

/* How dot products are accumulated by mmeb200_bgemm / mmeb200_conv from now on.
 *   MMEB200_ACC_TENSOR_CORE (default): tcgen05 tensor cores, fp32 accumulators; results agree with the reference's
 *       chip models within 1e-5 * sum|a_k b_k| per element.
 *   MMEB200_ACC_CHIP_EXACT: the reference's Gaudi3 arithmetic itself, on the GPU's integer units -- blocks of eight
 *       exact products plus the accumulator, aligned to the largest exponent with 24 + 4 truncated fraction bits,
 *       summed and truncated (chip_fma/gaudi3_fma.cpp:70-144,190-235 over fs_fma_gaudi3.h:760-1166): accumulators
 *       are bit-identical to CPUCalculator's. bf16 x bf16, fp8 x fp8 (any bias / Inf-NaN mode, mixed 143 / 152), and
 *       fp32 x fp32 / tf32 x tf32 through the chip's sliced multiplier (fs_fma_gaudi3.h:1820-1843, fs_fma.cpp:3546-3581),
 *       on a Gaudi3 context; convolutions run as im2col + GEMM (+ col2im), as the reference does; the cast is a
 *       separate pass. Three orders of magnitude slower than the tensor-core path (fp8 8192^3: 0.9 s against 0.37 ms) and
 *       three orders faster than the CPU reference on 16 host cores. */
enum { MMEB200_ACC_TENSOR_CORE = 0, MMEB200_ACC_CHIP_EXACT = 1 };
int mmeb200_set_accumulation(mmeb200_ctx* ctx, int mode);

/* Tuning knobs of a context; no counterpart in the reference (its calculator has limitNumOfThreads only). The planner
 * picks tile shapes, K splits and store paths per problem; a knob forces one choice, value < 0 gives it back to the
 * planner. Names: "pair" (0/1: CTA-pair kernel), "block_n" (128/256: single-CTA tile width), "split_k" (n > 0),
 * "epi_groups" (1/2), "raster_gm" (m tiles per raster group), "tma_store" (0 = direct stores), "host_pipeline"
 * (0 = host-tensor GEMMs staged whole), "tile_n" (CTA-pair kernel: tile width, a multiple of 32 up to 256), "stream_k"
 * (CTA-pair kernel: 1 = the tiles of a ragged last wave are cut along K among the CTA pairs wherever a cut exists; off by
 * default, it did not pay on the shapes measured), "dependent_launch" (0 = the tcgen05 GEMM kernels are launched without programmatic
 * stream serialisation; with it, the kernel's set-up overlaps the tail of the kernel before it in the stream and it touches
 * memory only after that kernel has completed). The same knobs take their defaults from environment variables read once in
 * mmeb200_create (MME_B200_PAIR, MME_B200_BLOCK_N, MME_B200_SPLIT_K, MME_B200_EPI_GROUPS, MME_B200_GM,
 * MME_B200_NO_TMA_STORE, MME_B200_NO_HOST_PIPELINE, MME_B200_TILE_N, MME_B200_STREAM_K, MME_B200_DEPENDENT_LAUNCH); no launch
 * reads the environment. Results do not depend on the knobs beyond the accumulation tolerance (summation order). */
int mmeb200_set_option(mmeb200_ctx* ctx, const char* name, int value);

/* Run all later work of this context on the caller's CUDA stream (a cudaStream_t passed as
 * void*); NULL goes back to the context's own stream. */
int mmeb200_set_stream(mmeb200_ctx* ctx, void* cuda_stream);

/* Replaces CPUCalculator::limitNumOfThreads (mme_reference_impl.cpp:2002-2012): kept for
 * signature compatibility, a no-op on the GPU. */
int mmeb200_limit_num_of_threads(mmeb200_ctx* ctx, unsigned n);

/* Replaces CPUCalculator::doBatchGemm (mme_reference_impl.cpp:445-539), and with 2-dim tensors
 * CPUCalculator::doGemm (:541-565). out->dtype == fp32 gives the reference's fp32 accumulator.
 * When `cast` is non-NULL the epilogue also does what doActivation would do next
 * (:661-689,1143-1245) and writes out->dtype directly (bf16 / fp8 / fp32). */
int mmeb200_bgemm(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_tensor* x,
                  const mmeb200_tensor* w, int op, const mmeb200_cast_params* cast);

/* Replaces CPUCalculator::doConvolution (mme_reference_impl.cpp:598-659): op is FWD, DEDX,
 * DEDW or TRANSPOSED_DEDX; `out` is y, x or w respectively. `rounding` reaches only the fp32
 * adds that merge filter taps in dedx (im2col.cpp:93-132). `cast` as in mmeb200_bgemm. */
int mmeb200_conv(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_tensor* x,
                 const mmeb200_tensor* w, const mmeb200_tensor* y,
                 const mmeb200_conv_params* params, int op, int rounding,
                 const mmeb200_cast_params* cast);

/* Replaces CPUCalculator::doActivation without ActivationParams (mme_reference_impl.cpp:661-689)
 * -> convertToOutputDataType (:1143-1245): optional ReLU on the fp32 accumulator (in place, as
 * the reference does), then the rounded cast. With rng_kind == MMEB200_RNG_LFSR the context's
 * LFSR registers are used and advanced exactly like m_lfsr in the reference. */
int mmeb200_activation(mmeb200_ctx* ctx, mmeb200_tensor* out, mmeb200_tensor* acc,
                       const mmeb200_cast_params* cast);

/* Replaces CPUCalculator::doMemoryWrite (mme_reference_impl.cpp:718-768): copy, or a
 * read-modify-write reduction of mme_out into mem (fp32 and bf16). */
int mmeb200_memory_write(mmeb200_ctx* ctx, mmeb200_tensor* mem, const mmeb200_tensor* mme_out,
                         int reduction_op, int reduction_rm, int clip_fp);

/* Bulk conversion utilities (the typed wrappers bf16_t / fp8_14x_t / fp32_t / tf32_t in
 * mme/mme_reference/data_types, over coral-sim/src/gaudi3/fs_core/fs_fma.cpp:851-924,
 * 6066-6140,6731-7029): fp8/bf16/tf32 -> fp32 decode, or fp32 -> any out dtype with `cast`. */
int mmeb200_convert(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_tensor* in,
                    const mmeb200_cast_params* cast);

/* Replaces CPUCalculator::doDma (mme_reference_impl.cpp:396-443): MEMCPY or TRANS (swap of the
 * two fastest dims); GEMM_TRANSPOSE is the same transposition. */
int mmeb200_dma(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_tensor* x, int op);

/* Read / overwrite the LFSR registers and polynomial (m_lfsr, m_polynomial,
 * mme_reference_impl.h:251-253). */
int mmeb200_get_lfsr(mmeb200_ctx* ctx, uint32_t* regs, uint32_t num_regs, uint32_t* polynomial);
int mmeb200_set_lfsr(mmeb200_ctx* ctx, const uint32_t* regs, uint32_t num_regs, uint32_t polynomial);

/* Wait, with a deadline, for everything queued on the context's stream; also collects the
 * status word of the bounded in-kernel waits. No counterpart in the reference (it is
 * synchronous); host-tensor calls sync internally. */
int mmeb200_sync(mmeb200_ctx* ctx, uint64_t timeout_ns);

/* Text of the last failure on this context (the message the shim hands to MME_ASSERT). */
const char* mmeb200_last_error(const mmeb200_ctx* ctx);

/* Device-memory helpers for callers that do not link the CUDA runtime (the benchmark and the
 * multi-GPU driver keep operands resident with these). No counterpart in the reference. */
int mmeb200_device_count(void);
int mmeb200_malloc(mmeb200_ctx* ctx, void** dev_ptr, size_t bytes);
int mmeb200_free(mmeb200_ctx* ctx, void* dev_ptr);
int mmeb200_memcpy_h2d(mmeb200_ctx* ctx, void* dev_dst, const void* host_src, size_t bytes);
int mmeb200_memcpy_d2h(mmeb200_ctx* ctx, void* host_dst, const void* dev_src, size_t bytes);
int mmeb200_memset(mmeb200_ctx* ctx, void* dev_dst, int value, size_t bytes);
/* Free and total device memory of the context's GPU (cudaMemGetInfo). */
int mmeb200_mem_info(mmeb200_ctx* ctx, size_t* free_bytes, size_t* total_bytes);
/* Pinned host staging memory, so host-tensor calls copy at full PCIe rate. */
int mmeb200_host_alloc(void** host_ptr, size_t bytes);
int mmeb200_host_free(void* host_ptr);

/* CUDA-event timing on the context's stream, for the benchmark: elapsed milliseconds between
 * two recorded marks. */
int mmeb200_timer_start(mmeb200_ctx* ctx);
int mmeb200_timer_stop(mmeb200_ctx* ctx, float* elapsed_ms);

/* No counterpart in the reference. A split-K GEMM for callers that must not allocate while they
 * run: code living under a framework's memory pool that was handed exactly its inputs and outputs,
 * a latency-critical loop that cannot afford the allocator's lock, a process whose device-memory
 * budget was fixed at start-up. out[M x N] (fp32) = op(x) . op(w) with the reduction cut into
 * `splits` parts whose fp32 partial sums live in a fixed 16 MiB array inside the library image
 * (held by every GPU that loads the library, until the process exits) instead of in scratch memory
 * from cudaMalloc. After the first call on a device (see below) a call performs no cudaMalloc / cudaFree
 * and calls no allocating routine: free device memory is the same before and after it.
 *   - tensors: device-resident, 2-D, 16-byte aligned, row pitches multiples of 16 bytes; bf16 x bf16,
 *     or fp8 whose Inf/NaN convention matches the tensor cores (1-4-3 minimal, 1-5-2 full);
 *   - limit: splits * M * N * 4 bytes <= 16 MiB, 2 <= splits <= 64; larger requests are rejected
 *     with MMEB200_ERR_INVALID_ARG and a message naming the limit;
 *   - the first call on a device does the one-time set-up: it looks up the array's device address
 *     (cudaGetSymbolAddress), sets the kernel's shared-memory attribute, resolves the driver's
 *     tensor-map encoder, and the CUDA runtime loads the kernels' module on first use. Make that
 *     warm-up call where allocation is still allowed, and before any stream capture;
 *   - all calls share the one array and it keeps the previous call's partial sums. Each call
 *     overwrites every element it later reads, so nothing needs clearing, but two calls that
 *     overlap on the GPU (different streams or contexts) race on it: serialise them. */
int mmeb200_gemm_splitk_static(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_tensor* x,
                               const mmeb200_tensor* w, int op, int splits);

/* Replaces TensorComparator::doCompare / doCompareBitExact (mme/mme_reference/tensor_comparator.h:13-43,
 * rule in tensor_comparator_impl.cpp:372-438,578-592) for dense tensors: `a` holds num_partials stacked
 * results (summed in fp32 and rounded to the element type when num_partials > 1; fp32 and bf16 only),
 * `b` the tensor compared with; dtype, exponent bias and Inf/NaN mode are b's. cd_size is the common
 * dimension (sets the ULP allowance). Returns the number of mismatching elements and the lowest
 * mismatching flat index (valid when mismatches != 0). */
typedef struct mmeb200_compare_result {
    uint64_t mismatches;
    uint64_t first_index;
} mmeb200_compare_result;
int mmeb200_compare(mmeb200_ctx* ctx, const mmeb200_tensor* a, const mmeb200_tensor* b, unsigned cd_size,
                    unsigned num_partials, int bit_exact, mmeb200_compare_result* result);

/* Replaces RandomSimTensorGenerator::generateUniform / generateNormal / fill / generateUnitMatrix /
 * fillForReductionPacking (mme/mme_reference/sim_tensor.h:108-166, sim_tensor.cpp:100-191): fills a dense tensor
 * on the device. min_value / max_value are first clamped to the finite range of the tensor's type, bias and
 * Inf/NaN mode (sim_tensor.cpp:116-119); normal draws are clamped to that range; values are rounded to the type
 * with round-to-nearest-even. UNIT writes max_value to the first element and min_value to the rest, as the
 * reference does. The random stream is Philox4x32-10 keyed by (seed, element index): the same distributions as the
 * reference, not its mt19937 sequence, so both sides of a comparison must be fed from this one buffer. */
enum {
    MMEB200_GEN_UNIFORM = 0,
    MMEB200_GEN_NORMAL = 1,
    MMEB200_GEN_FILL = 2,             /* every element = min_value */
    MMEB200_GEN_UNIT = 3,
    MMEB200_GEN_REDUCTION_PACKING = 4 /* element (row, col) = 1 when row == col % packing, rows of packing * level */
};
typedef struct mmeb200_generate_params {
    int32_t kind;
    float min_value, max_value, mean, std_dev;
    uint32_t packing, level;
    uint64_t seed;
} mmeb200_generate_params;
int mmeb200_generate(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_generate_params* params);

/* ---- dedw across the GPUs of one box, reduction fused with the exchange --------------------------
 * The reference sums partial weight gradients with doMemoryWrite's fp32 add
 * (mme_reference_impl.cpp:718-768; partial tensors: mme_verification/common/mme_test_manager.cpp:655-690).
 * Here every rank (one process per GPU) computes dW over its images, and the exchange is a reduce-scatter
 * followed by an all-gather over peer memory, fused with the split-K reduction: the kernel that reduces the
 * K-splits stores every element straight into the exchange buffer of the element's OWNER rank over NVLink
 * (plain peer stores; nothing loads from a peer), each owner adds the `world` partials of its 1/world of dW
 * in rank order and stores the sums to every rank: all ranks end with bit-identical sums, no host round
 * trip, no separate collective, and 2 * (world-1)/world of dW leaves each rank. Every wait is bounded.
 * Exchange buffers (mmeb200_peer_exchange_bytes) and flag blocks (256 bytes) are allocated with
 * mmeb200_peer_alloc, their handles exchanged by the caller (any transport) and opened with mmeb200_peer_open. */
#define MMEB200_MAX_PEERS 8
#define MMEB200_PEER_HANDLE_BYTES 64
typedef struct mmeb200_peer_group {
    int32_t rank, world;                 /* 1 <= world <= 8 */
    void* slots[MMEB200_MAX_PEERS];      /* slots[j]: rank j's exchange buffer (mmeb200_peer_exchange_bytes), addressable from this GPU */
    uint32_t* flags[MMEB200_MAX_PEERS];  /* flags[j]: rank j's flag block (256 bytes, zero before the first exchange) */
    uint32_t step;                       /* exchanges already done on this (slots, flags) set */
    uint32_t deferred_output;            /* non-zero (device `out` only): the owner's sum and the final copy run on a side
                                            stream and overlap the next call's convolution; `out` is complete after the
                                            next mmeb200_sync, and is ordered before the next exchange's output */
} mmeb200_peer_group;
/* Bytes of one rank's exchange buffer for a result of n_floats fp32 values shared by `world` ranks: `world` partial
 * slots of the rank's own segment plus the assembled result. */
size_t mmeb200_peer_exchange_bytes(uint64_t n_floats, int world);
/* cudaMalloc'd, zero-filled device memory plus the handle other processes open it with. */
int mmeb200_peer_alloc(mmeb200_ctx* ctx, size_t bytes, void** dev_ptr, unsigned char handle[MMEB200_PEER_HANDLE_BYTES]);
int mmeb200_peer_open(mmeb200_ctx* ctx, const unsigned char handle[MMEB200_PEER_HANDLE_BYTES], void** dev_ptr);
int mmeb200_peer_close(mmeb200_ctx* ctx, void* dev_ptr);
/* doConvolution(dedw) over this rank's x / y, summed over all ranks of `group` into `out` (fp32, dense,
 * the full dW; its element count must be a multiple of 4). Consecutive calls must alternate between two (slots, flags)
 * sets so that a fast rank cannot overwrite slots a slow rank still reads; `step` counts the calls made on the set passed.
 * Works in either accumulation mode (the bit-exact mode exchanges its exact partials the same way).
 * A rank that waits longer than about a second for its peers gets MMEB200_ERR_DEVICE_WAIT from the next
 * mmeb200_sync and stays usable. */
int mmeb200_conv_dedw_allreduce(mmeb200_ctx* ctx, mmeb200_tensor* out, const mmeb200_tensor* x,
                                const mmeb200_tensor* w, const mmeb200_tensor* y,
                                const mmeb200_conv_params* params, const mmeb200_peer_group* group);

/* Number of kernels this library has launched on the context since creation. */
uint64_t mmeb200_launch_count(const mmeb200_ctx* ctx);

/* Library version string, e.g. "mme_b200 0.1 sm_100a". */
const char* mmeb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MME_B200_H */
