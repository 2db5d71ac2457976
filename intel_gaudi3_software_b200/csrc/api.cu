// C ABI of libmme_b200.so (see include/mme_b200.h): context, host<->device staging, operand
// planning (tensor maps, repacking, split-K, conv lowering choice) and kernel launches.
// There is no CPU compute path in this file: every operation either runs on the GPU or fails.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "gemm_launch.h"
#include "gemm_sm100.cuh"
#include "gaudi3_exact.cuh"
#include "kernels.cuh"
#include "mme_b200.h"

using namespace mmeb200;

// ------------------------------------------------------------------------------------------ context
struct ArenaBlock {
    void* ptr;
    size_t size, used;
};

// Tuning knobs of a context (-1 = let the planner decide). Their defaults come from the environment ONCE, when the
// context is created (MME_B200_PAIR, _BLOCK_N, _SPLIT_K, _EPI_GROUPS, _GM, _NO_TMA_STORE, _NO_HOST_PIPELINE, _TILE_N);
// mmeb200_set_option changes them per context afterwards. No launch reads the environment.
struct Tuning {
    int pair = -1;            // 0 / 1: CTA-pair kernel off / on where it applies
    int block_n = -1;         // 128 / 256: single-CTA tile width (turns the pair kernel off)
    int split_k = -1;         // > 0: forced number of K splits
    int epi_groups = -1;      // 1 / 2: groups of four epilogue warps in the pair kernel
    int raster_gm = -1;       // m tiles per raster group
    int tma_store = -1;       // 0: direct stores even where a TMA store applies
    int host_pipeline = -1;   // 0: host-tensor GEMMs are staged whole instead of pipelined
    int tile_n = -1;          // CTA-pair kernel: forced tile width (a multiple of 32 in [32, 256])
    int stream_k = -1;        // 1: cut the tiles of a ragged last wave along K (CTA-pair kernel) whenever a cut exists
    int dependent_launch = -1;   // 0: the CTA-pair kernel is launched without programmatic stream serialisation
};
static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

struct mmeb200_ctx {
    int device = 0, chip = 2, sm_count = 148;
    Tuning tune;
    unsigned seed = 0;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    std::string err;
    std::vector<ArenaBlock> arena;
    uint32_t* d_status = nullptr;
    uint32_t* h_status = nullptr;  // pinned
    std::vector<uint32_t> lfsr;
    uint32_t polynomial = 0;
    uint32_t* d_jump = nullptr;    // 32 x 32 words: column images of M^(2^j)
    uint32_t jump_poly = 0;
    std::vector<uint32_t> h_jump;
    uint32_t* d_lfsr = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    const mmeb200_peer_group* pending_peer = nullptr;   // set by mmeb200_conv_dedw_allreduce for the next GEMM
    cudaStream_t s_h2d = nullptr, s_d2h = nullptr;   // copy streams of the pipelined host-tensor GEMM
    cudaEvent_t ev_in[17] = {}, ev_done[17] = {};
    int acc_mode = 0;   // MMEB200_ACC_*
    // deferred output of the fused dedw exchange: the wait-and-add kernel runs here
    cudaStream_t s_side = nullptr;
    cudaEvent_t ev_scatter = nullptr, ev_gather = nullptr;
    bool gather_pending = false;
    uint64_t launches = 0;
    void* aux = nullptr;            // dense copies of strided convolution tensors (outlives the per-call arena)
    size_t aux_bytes = 0;
    // cut tail of the CTA-pair kernel: slots for the partial sums of the cut tiles' pieces, one flag word per epilogue warp and slot
    float* sk_ws = nullptr;
    uint32_t* sk_flags = nullptr;
    uint32_t sk_slots_cap = 0, sk_gen = 0;

    int fail(int code, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        err = buf;
        return code;
    }
};

#define CUDA_OK(ctx, call)                                                                            \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess) return (ctx)->fail(MMEB200_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)
#define TRY(expr)              \
    do {                       \
        int rc_ = (expr);      \
        if (rc_ != 0) return rc_; \
    } while (0)

static thread_local std::string g_static_err;

// Scratch memory: bump-allocated blocks, recycled at the start of every API call. Work of one
// context is ordered on one stream, so a block may be reused while earlier kernels still run.
static void arena_reset(mmeb200_ctx* c) {
    if (c->arena.size() > 1) {
        size_t total = 0;
        cudaStreamSynchronize(c->stream);
        for (auto& b : c->arena) {
            total += b.size;
            cudaFree(b.ptr);
        }
        c->arena.clear();
        void* p = nullptr;
        if (cudaMalloc(&p, total) == cudaSuccess) c->arena.push_back({p, total, 0});
    }
    for (auto& b : c->arena) b.used = 0;
}
static int arena_alloc(mmeb200_ctx* c, void** out, size_t bytes) {
    bytes = (bytes + 1023) & ~size_t(1023);
    if (bytes == 0) bytes = 1024;
    for (auto& b : c->arena) {
        if (b.size - b.used >= bytes) {
            *out = static_cast<char*>(b.ptr) + b.used;
            b.used += bytes;
            return 0;
        }
    }
    size_t sz = std::max(bytes, size_t(64) << 20);
    void* p = nullptr;
    CUDA_OK(c, cudaMalloc(&p, sz));
    c->arena.push_back({p, sz, bytes});
    *out = p;
    return 0;
}

static inline unsigned grid_for(uint64_t n, int threads, int sm_count) {
    uint64_t blocks = (n + threads - 1) / threads;
    uint64_t cap = uint64_t(sm_count) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return unsigned(blocks);
}

// ------------------------------------------------------------------------------------------ tensors
static bool dtype_ok(int dt) {
    return dt == DT_FP8_143 || dt == DT_FP8_152 || dt == DT_BF16 || dt == DT_FP32 || dt == DT_FP32_IEEE || dt == DT_TF32;
}
static uint64_t num_elems(const mmeb200_tensor* t) {
    uint64_t n = 1;
    for (int d = 0; d < 5; ++d) n *= t->sizes[d];
    return n;
}
static uint64_t span_elems(const mmeb200_tensor* t) {
    if (num_elems(t) == 0) return 0;
    uint64_t s = 1;
    for (int d = 0; d < 5; ++d) s += uint64_t(t->sizes[d] - 1) * t->strides[d];
    return s;
}
static bool is_dense(const mmeb200_tensor* t) {
    uint64_t acc = 1;
    for (int d = 0; d < 5; ++d) {
        if (t->sizes[d] != 1 && t->strides[d] != acc) return false;
        acc *= t->sizes[d];
    }
    return true;
}
static int check_tensor(mmeb200_ctx* c, const mmeb200_tensor* t, const char* name) {
    if (!t) return c->fail(MMEB200_ERR_INVALID_ARG, "%s: null tensor", name);
    if (t->dims < 1 || t->dims > 5) return c->fail(MMEB200_ERR_INVALID_ARG, "%s: dims %d out of range", name, t->dims);
    if (!dtype_ok(t->dtype)) return c->fail(MMEB200_ERR_UNSUPPORTED, "%s: data type %d is not supported by this backend", name, t->dtype);
    if (t->strides[0] != 1) return c->fail(MMEB200_ERR_INVALID_ARG, "%s: strides[0] must be 1", name);
    if (num_elems(t) != 0 && !t->data) return c->fail(MMEB200_ERR_INVALID_ARG, "%s: null data", name);
    if (span_elems(t) >= (uint64_t(1) << 31)) return c->fail(MMEB200_ERR_UNSUPPORTED, "%s: tensors of 2^31 elements or more are not supported", name);
    return 0;
}

struct Staged {
    mmeb200_tensor t;  // data points to device memory
    void* host = nullptr;
    size_t bytes = 0;
};
// Bring a tensor's bytes to the device (no-op for device tensors).
static int stage_in(mmeb200_ctx* c, const mmeb200_tensor* src, Staged* s, bool copy_contents) {
    s->t = *src;
    s->host = nullptr;
    s->bytes = span_elems(src) * dtype_size(src->dtype);
    if (src->mem_space == MMEB200_MEM_DEVICE) return 0;
    void* d = nullptr;
    TRY(arena_alloc(c, &d, s->bytes));
    if (copy_contents && s->bytes) CUDA_OK(c, cudaMemcpyAsync(d, src->data, s->bytes, cudaMemcpyHostToDevice, c->stream));
    s->t.data = d;
    s->t.mem_space = MMEB200_MEM_DEVICE;
    s->host = src->data;
    return 0;
}
static int stage_out(mmeb200_ctx* c, Staged* s) {
    if (s->host && s->bytes) CUDA_OK(c, cudaMemcpyAsync(s->host, s->t.data, s->bytes, cudaMemcpyDeviceToHost, c->stream));
    return 0;
}

static int collect_status(mmeb200_ctx* c) {
    if (c->gather_pending) {   // a deferred exchange output: everything after this point is ordered behind it
        CUDA_OK(c, cudaStreamWaitEvent(c->stream, c->ev_gather, 0));
        c->gather_pending = false;
    }
    CUDA_OK(c, cudaMemcpyAsync(c->h_status, c->d_status, 4, cudaMemcpyDeviceToHost, c->stream));
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    if (*c->h_status != 0) {
        uint32_t code = *c->h_status;
        cudaMemsetAsync(c->d_status, 0, 4, c->stream);
        return c->fail(MMEB200_ERR_DEVICE_WAIT, "a bounded in-kernel wait gave up (code %u)", code);
    }
    return 0;
}
// Host-tensor calls are synchronous like the reference; device-tensor calls stay asynchronous.
static int finish_call(mmeb200_ctx* c, bool any_host) {
    CUDA_OK(c, cudaGetLastError());
    if (any_host) return collect_status(c);
    return 0;
}

// ------------------------------------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;
static int load_driver_entry_points(mmeb200_ctx* c) {
    if (g_encode_tiled && g_encode_im2col) return 0;
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    CUDA_OK(c, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn) return c->fail(MMEB200_ERR_CUDA, "driver does not export cuTensorMapEncodeTiled");
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    fn = nullptr;
    CUDA_OK(c, cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q));
    if (!fn) return c->fail(MMEB200_ERR_CUDA, "driver does not export cuTensorMapEncodeIm2col");
    g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
    return 0;
}
static CUtensorMapDataType tma_dtype(int elem) {
    return elem == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
}

// A GEMM operand as the kernel wants it: a 2-D view (inner x rows) plus three batch dims.
struct TmaOperand {
    const void* ptr = nullptr;
    int elem = 2;
    bool mn_major = false;       // inner dimension is M/N (true) or K (false)
    uint64_t inner = 0, rows = 0;
    uint64_t row_stride = 0;     // elements
    uint32_t bsz[3] = {1, 1, 1};
    uint64_t bstride[3] = {0, 0, 0};
    uint32_t hw_fmt = 0;
};

static bool tma_compatible(const TmaOperand& o) {
    if (reinterpret_cast<uintptr_t>(o.ptr) & 15) return false;
    if (o.rows > 1 && (o.row_stride * o.elem) % 16) return false;
    for (int i = 0; i < 3; ++i)
        if (o.bsz[i] > 1 && (o.bstride[i] * o.elem) % 16) return false;
    return true;
}

static int encode_tiled(mmeb200_ctx* c, CUtensorMap* tm, const TmaOperand& o, uint32_t box_inner, uint32_t box_rows, int u16_type = 0) {
    TRY(load_driver_entry_points(c));
    cuuint64_t dims[5] = {o.inner, o.rows, o.bsz[0], o.bsz[1], o.bsz[2]};
    cuuint64_t strides[4];
    uint64_t dense = std::max<uint64_t>(o.inner * o.elem, 16);
    dense = (dense + 15) & ~uint64_t(15);
    strides[0] = (o.rows > 1) ? o.row_stride * o.elem : dense;
    uint64_t prev = strides[0] * std::max<uint64_t>(o.rows, 1);
    for (int i = 0; i < 3; ++i) {
        strides[i + 1] = (o.bsz[i] > 1) ? o.bstride[i] * o.elem : ((prev + 15) & ~uint64_t(15));
        prev = strides[i + 1] * o.bsz[i];
    }
    cuuint32_t box[5] = {box_inner, box_rows, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    // 16-bit outputs are raw bit patterns: describe them as integers so the copy engine cannot touch them
    const CUtensorMapDataType dt = (u16_type == 2) ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : tma_dtype(o.elem);
    CUresult r = g_encode_tiled(tm, dt, 5, const_cast<void*>(o.ptr), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return c->fail(MMEB200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d): inner %llu rows %llu stride %llu box %u x %u", int(r),
                       (unsigned long long) o.inner, (unsigned long long) o.rows, (unsigned long long) strides[0], box_inner, box_rows);
    return 0;
}

// ------------------------------------------------------------------------------------------ GEMM launch
struct OutSpec {
    void* ptr;
    int dtype;
    uint64_t ld;
    uint32_t bsz[3];
    uint64_t bstride[3];
    float scale;
    bool has_cast;
    CastSpec cast;
    bool philox;
    uint64_t seed, offset;
};

static int launch_status(mmeb200_ctx* c, const LaunchResult& r) {
    if (r.cuda != cudaSuccess) return c->fail(MMEB200_ERR_CUDA, "%s: %s", r.what, cudaGetErrorString(r.cuda));
    if (r.code != LAUNCH_OK) return c->fail(MMEB200_ERR_CUDA, "%s", r.what);
    c->launches++;
    return 0;
}
static LaunchEnv launch_env(const mmeb200_ctx* c) { return LaunchEnv{c->device, c->sm_count, c->stream, c->tune.dependent_launch != 0}; }

struct GemmJob {
    TmaOperand a, b;
    bool a_im2col = false;
    CUtensorMap a_map;       // pre-encoded when a_im2col
    ConvGeom conv = {};
    uint32_t M = 0, N = 0, K = 0;
    uint32_t kind = KIND_F16;
    uint32_t bsz[3] = {1, 1, 1};   // output batch dims
    int force_split = 0;
    const uint32_t* pred = nullptr;   // device-side predicate of this form of the GEMM (GemmParams::pred)
    uint32_t pred_nonzero = 0;
};

static uint64_t peer_segment_floats(uint64_t n, int world) {
    const uint64_t n4 = (n + 3) / 4;
    return ((n4 + uint64_t(world) - 1) / uint64_t(world)) * 4;
}

// The cross-GPU sum of one fp32 result (dedw's partial dW): `splits` partial copies of n floats in `ws` are summed,
// reduce-scattered to their owner ranks, summed there in rank order and all-gathered into `out` on every rank
// (kernels.cuh: splitk_reduce_peer_scatter_kernel, peer_owner_sum_kernel, peer_result_copy_kernel).
static int run_peer_exchange(mmeb200_ctx* c, const mmeb200_peer_group* peer, const float* ws, uint32_t splits, uint64_t n, float scale,
                             float* out) {
    if (n % 4) return c->fail(MMEB200_ERR_UNSUPPORTED, "the fused dedw exchange needs a result whose size is a multiple of 4");
    const uint64_t seg = peer_segment_floats(n, peer->world);
    PeerScatter ps;
    memset(&ps, 0, sizeof ps);
    PeerOwnerSum po;
    memset(&po, 0, sizeof po);
    for (int i = 0; i < peer->world; ++i) {
        ps.bufs[i] = po.bufs[i] = static_cast<float*>(peer->slots[i]);
        ps.flags[i] = po.flags[i] = peer->flags[i];
    }
    ps.block_counter = c->d_status + 8;
    ps.rank = peer->rank; ps.world = peer->world; ps.splits = splits; ps.n = n; ps.seg = seg; ps.scale = scale;
    po.block_counter = c->d_status + 9;
    po.rank = peer->rank; po.world = peer->world; po.n = n; po.seg = seg;
    po.target = uint32_t(peer->world) * (peer->step + 1);
    po.status = c->d_status; po.limit_ns = 1000000000ull;
    PeerResultCopy pc;
    memset(&pc, 0, sizeof pc);
    pc.my_buf = static_cast<const float*>(peer->slots[peer->rank]);
    pc.my_flags = peer->flags[peer->rank];
    pc.target = po.target; pc.world = peer->world; pc.n = n; pc.seg = seg; pc.out = out;
    pc.status = c->d_status; pc.limit_ns = 1000000000ull;
    const unsigned blocks = grid_for(n / 4, 256, c->sm_count);
    const unsigned owner_blocks = grid_for(seg / 4, 256, c->sm_count);
    const bool deferred = peer->deferred_output != 0;
    // The exchange kernels are meant to share the SMs with the next convolution's GEMM, whose CTAs configure the SM for
    // the largest shared-memory carve-out: blocks of kernels that ask for different carve-outs do not run on an SM together,
    // so these ask for the same one.
    static bool carveout_set[64] = {};
    if (!carveout_set[c->device & 63]) {
        CUDA_OK(c, cudaFuncSetAttribute(splitk_reduce_peer_scatter_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        CUDA_OK(c, cudaFuncSetAttribute(peer_owner_sum_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        CUDA_OK(c, cudaFuncSetAttribute(peer_result_copy_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        carveout_set[c->device & 63] = true;
    }
    if (deferred && !c->s_side) {
        CUDA_OK(c, cudaStreamCreateWithFlags(&c->s_side, cudaStreamNonBlocking));
        CUDA_OK(c, cudaEventCreateWithFlags(&c->ev_scatter, cudaEventDisableTiming));
        CUDA_OK(c, cudaEventCreateWithFlags(&c->ev_gather, cudaEventDisableTiming));
    }
    // A rank may announce exchange i+1 only after it has read its buffers of exchange i: the partners' next-but-one stores
    // reuse them, and they are held back only by this rank's arrivals.
    if (c->gather_pending) CUDA_OK(c, cudaStreamWaitEvent(c->stream, c->ev_gather, 0));
    splitk_reduce_peer_scatter_kernel<<<blocks, 256, 0, c->stream>>>(ws, ps);
    cudaStream_t tail = c->stream;
    if (deferred) {
        CUDA_OK(c, cudaEventRecord(c->ev_scatter, c->stream));
        CUDA_OK(c, cudaStreamWaitEvent(c->s_side, c->ev_scatter, 0));
        tail = c->s_side;
    }
    peer_owner_sum_kernel<<<owner_blocks, 256, 0, tail>>>(po);
    peer_result_copy_kernel<<<blocks, 256, 0, tail>>>(pc);
    if (deferred) CUDA_OK(c, cudaEventRecord(c->ev_gather, c->s_side));
    c->gather_pending = deferred;
    c->launches += 3;
    CUDA_OK(c, cudaGetLastError());
    return 0;
}

static int run_gemm(mmeb200_ctx* c, GemmJob& j, const OutSpec& o) {
    GemmParams p;
    memset(&p, 0, sizeof p);
    const int elem = j.b.elem;
    p.M = j.M; p.N = j.N; p.K = j.K;
    p.elem_bytes = elem;
    p.block_k = kRowBytes / elem;
    p.num_k_blocks = (j.K + p.block_k - 1) / p.block_k;
    p.m_tiles = (j.M + kBlockM - 1) / kBlockM;
    p.batches = j.bsz[0] * j.bsz[1] * j.bsz[2];
    for (int i = 0; i < 3; ++i) {
        p.bsz[i] = j.bsz[i];
        p.a_bcast[i] = (j.a.bsz[i] == 1);
        p.b_bcast[i] = (j.b.bsz[i] == 1);
        p.out_bstride[i] = o.bstride[i];
    }
    p.a_mn_major = j.a.mn_major;
    p.b_mn_major = j.b.mn_major;
    p.a_mode = j.a_im2col ? A_IM2COL : A_TILED;
    p.conv = j.conv;
    // Tile geometry. CTA pairs (one 256 x 256 tile per two SMs, half the B traffic per SM) whenever the
    // problem is at least one such tile; else 128 x 256 tiles per CTA whenever N has the columns; else
    // 128 x 128. Split-K below fills the machine when that leaves few tiles.
    const Tuning& tune = c->tune;
    bool use_pair = j.M >= 256 && j.N >= 256;
    if (tune.pair >= 0) use_pair = use_pair && tune.pair != 0;
    const bool wide = j.N > 128;
    int block_n = wide ? 256 : 128;
    if (tune.block_n >= 0) { block_n = tune.block_n == 256 ? 256 : 128; use_pair = false; }
    uint64_t tiles, units;   // units = CTAs or CTA pairs the device runs at once
    uint32_t tile_n = 256;
    if (use_pair) {
        p.m_tiles = (j.M + 255) / 256;
        block_n = 128;       // each CTA stages (up to) 128 of the pair's columns of B
        units = uint64_t(gemm_pair_capacity(launch_env(c), j.kind, 1));
        if (units == 0) units = uint64_t(c->sm_count) / 2;
        // Tile width: 256 unless the knob narrows it. Narrower tiles would fill a ragged last wave better (8192-wide outputs
        // with 1024 rows: 4 x 37 tiles of 224 are exactly two waves of 74 pairs), but measured they lose: at 256 columns a
        // k block's MMAs take as long as its 32 KB of operands take to arrive, so a narrower tile, which moves the same A
        // for fewer columns, is bound by the operand feed (fp8 1024 x 8192 x 8192: 62 us at 256, 75 us at 224, 102 us at 128).
        if (tune.tile_n > 0) tile_n = std::min(256, std::max(32, (tune.tile_n / 32) * 32));
        p.n_tiles = (j.N + tile_n - 1) / tile_n;
    } else {
        p.n_tiles = (j.N + block_n - 1) / block_n;
        units = uint64_t(c->sm_count);
    }
    p.tile_n = tile_n;
    p.raster_gm = plan_raster_group(use_pair ? 256 : kBlockM, j.K, uint32_t(elem));   // schedule.cuh
    if (tune.raster_gm > 0) p.raster_gm = tune.raster_gm;
    tiles = uint64_t(p.m_tiles) * p.n_tiles * p.batches;
    uint32_t split = 1;
    if (j.conv.out_grid) j.force_split = 1;   // the split-K reduction writes rows out_ld apart; a parity class does not
    else if (tune.split_k > 0) j.force_split = tune.split_k;
    if (j.force_split > 0) split = std::min<uint32_t>(j.force_split, p.num_k_blocks);
    else if (tiles * 2 <= units && p.num_k_blocks >= 32) {
        // worth it only when the k loop is long: the partial sums cost a second kernel and (splits + 1) passes over M x N floats
        split = uint32_t(std::min<uint64_t>(units / tiles, p.num_k_blocks / 8));
        split = std::max(1u, std::min(split, 64u));
    }
    // no empty splits
    while (split > 1 && ((p.num_k_blocks + split - 1) / split) * (split - 1) >= p.num_k_blocks) --split;
    // A small problem that is not split and would leave most SMs idle runs as 128 x 128 tiles: half the work per SM
    // on up to four times as many SMs (1024^3 bf16: 11.5 us instead of 14.4 us).
    if (split == 1 && tune.block_n < 0 && tune.pair < 0) {
        const uint64_t sms_used = use_pair ? tiles * 2 : tiles;
        const uint64_t t128 = uint64_t((j.M + 127) / 128) * ((j.N + 127) / 128) * p.batches;
        if (sms_used * 2 <= uint64_t(c->sm_count) && t128 <= uint64_t(c->sm_count) && t128 > sms_used) {
            use_pair = false;
            block_n = 128;
            p.m_tiles = (j.M + kBlockM - 1) / kBlockM;
            p.n_tiles = (j.N + 127) / 128;
            tiles = t128;
        }
    }
    p.split_k = split;
    p.idesc = use_pair ? make_instr_desc(j.a.hw_fmt, j.b.hw_fmt, j.a.mn_major, j.b.mn_major, 256, tile_n)
                       : make_instr_desc(j.a.hw_fmt, j.b.hw_fmt, j.a.mn_major, j.b.mn_major, kBlockM, block_n);
    p.status = c->d_status;
    p.pred = j.pred;
    p.pred_nonzero = j.pred_nonzero;
    p.scale = o.scale;
    p.out_dtype = o.dtype;
    p.has_cast = o.has_cast;
    p.cast = o.cast;
    if (!o.has_cast) p.epi_mode = EPI_F32;
    else if (o.cast.out_dtype == DT_BF16 && o.cast.rm == RM_NE && !o.cast.relu && !o.cast.clip && !o.cast.ftz) p.epi_mode = EPI_BF16_RNE;
    else if (o.cast.out_dtype == DT_FP32 && !o.cast.relu && !o.cast.clip && !o.cast.ftz) p.epi_mode = EPI_F32;
    else if (cast_is_fp8_hw(o.cast)) {
        // the output's Inf/NaN convention is the hardware fp8 format's: saturating hardware conversion after an exact rescale
        p.epi_mode = EPI_FP8_HW;
        p.hw = fp8_hw_cast(o.cast);
    } else p.epi_mode = EPI_GENERIC;
    p.rng_philox = o.philox;
    p.rng_seed = o.seed;
    p.rng_offset = o.offset;
    p.out_ld = o.ld;
    p.out = o.ptr;
    void* ws = nullptr;
    const mmeb200_peer_group* peer = c->pending_peer;
    c->pending_peer = nullptr;
    if (peer && j.pred) return c->fail(MMEB200_ERR_UNSUPPORTED, "the fused dedw exchange takes operands whose fp8 convention the tensor cores share");
    if (peer) {
        // the raw fp32 partial(s) go to scratch; the peer kernels below finish the job
        if (p.batches != 1 || o.has_cast || (uint64_t(j.M) * j.N) % 4)
            return c->fail(MMEB200_ERR_UNSUPPORTED, "the fused dedw exchange needs a single fp32 result whose size is a multiple of 4");
        if (o.dtype != DT_FP32) return c->fail(MMEB200_ERR_UNSUPPORTED, "the fused dedw exchange sums fp32 results");
        TRY(arena_alloc(c, &ws, size_t(split) * j.M * j.N * 4));
        p.out = ws;
        if (split == 1) { p.out_ld = j.N; p.scale = 1.0f; p.epi_mode = EPI_F32; p.has_cast = 0; p.out_dtype = DT_FP32; }
    } else if (split > 1) {
        TRY(arena_alloc(c, &ws, size_t(split) * p.batches * j.M * j.N * 4));
        p.out = ws;
    }
    // a tile with few k blocks spends longer in its epilogue than in its MMAs: give it eight epilogue warps; and so does
    // the general cast (stochastic rounding, fp8 output), tens of instructions per element
    bool two_groups = (p.num_k_blocks + split - 1) / split <= 12 || (split == 1 && (p.epi_mode == EPI_GENERIC || p.epi_mode == EPI_FP8_HW));
    if (tune.epi_groups > 0) two_groups = tune.epi_groups == 2;
    if (use_pair) {   // plan with what both variants of the pair kernel hold at once
        const uint64_t cap2 = uint64_t(gemm_pair_capacity(launch_env(c), j.kind, 2));
        if (cap2) units = std::min(units, cap2);
    }
    // Cut tail: with whole tiles only, `tiles % units` tiles make a last wave that leaves pairs idle (1024 x 8192 outputs:
    // 128 tiles on 74 pairs, 1.73 waves). Each of those tiles can be cut along K into a head, computed by a pair of its own,
    // and pieces that the remaining pairs share; the head's pair adds the pieces' sums and finishes the tile (PairSchedule and
    // plan_cut_tail, schedule.cuh). Head and piece lengths are the ones that finish earliest by a cost model in k blocks. Measured,
    // the cut does not pay on this part (a ragged wave runs its k blocks faster, the kernel being bound by the aggregate
    // L2-to-SM operand rate; a piece's sums cost 128 KB per CTA written and read again beside that stream): it is taken
    // only when the knob "stream_k" asks for it.
    uint64_t launch_pairs = tiles * split;
    if (use_pair && split == 1 && !peer && tune.stream_k > 0 && units > 1) {
        const uint64_t rem = tiles % units;
        const uint32_t nkb = p.num_k_blocks;
        const CutPlan cut = plan_cut_tail(rem, units, nkb, true);
        const uint32_t best_head = cut.head, best_piece = cut.piece, best_pieces = cut.pieces;
        if (best_head) {
            // eight epilogue warps: adding a slot's sums is bound by the loads a warp keeps in flight (the cut-tail kernel
            // exists in that form only)
            two_groups = true;
            const uint32_t slots = uint32_t(rem) * best_pieces;
            if (c->sk_slots_cap < slots) {
                if (c->sk_ws) { CUDA_OK(c, cudaStreamSynchronize(c->stream)); cudaFree(c->sk_ws); cudaFree(c->sk_flags); c->sk_ws = nullptr; c->sk_flags = nullptr; }
                const uint32_t cap = std::max(slots, 74u);
                CUDA_OK(c, cudaMalloc(&c->sk_ws, size_t(cap) * 2 * kSkSlotFloats * sizeof(float)));
                CUDA_OK(c, cudaMalloc(&c->sk_flags, size_t(cap) * 2 * kSkFlagsPerCta * sizeof(uint32_t)));
                CUDA_OK(c, cudaMemsetAsync(c->sk_flags, 0, size_t(cap) * 2 * kSkFlagsPerCta * sizeof(uint32_t), c->stream));
                c->sk_slots_cap = cap;
                c->sk_gen = 0;
            }
            p.sk_tiles = uint32_t(rem);
            p.sk_head = best_head;
            p.sk_piece = best_piece;
            p.sk_pieces = best_pieces;
            p.sk_ws = c->sk_ws;
            p.sk_flags = c->sk_flags;
            p.sk_gen = ++c->sk_gen;
            launch_pairs = units;   // heads on the first pairs, pieces on the others
        }
    }
    if (j.a_im2col) p.tm_a = j.a_map;
    else if (!j.a.mn_major) TRY(encode_tiled(c, &p.tm_a, j.a, p.block_k, kBlockM));
    else TRY(encode_tiled(c, &p.tm_a, j.a, kRowBytes / elem, p.block_k));
    // B per CTA: block_n columns, or half a narrowed pair tile (whole 128-byte groups when N is the contiguous dimension)
    const uint32_t b_cols = use_pair ? tile_n / 2 : uint32_t(block_n);
    if (!j.b.mn_major) {
        TRY(encode_tiled(c, &p.tm_b, j.b, p.block_k, b_cols));
        p.b_cta_bytes = b_cols * kRowBytes;
    } else {
        TRY(encode_tiled(c, &p.tm_b, j.b, kRowBytes / elem, p.block_k));
        p.b_cta_bytes = ((b_cols * elem + kRowBytes - 1) / kRowBytes) * p.block_k * kRowBytes;
    }
    // coalesced TMA stores when the output's base and pitches allow a tensor map
    if (split == 1 && !peer && tune.tma_store != 0 && !j.conv.out_grid) {
        TmaOperand od;
        od.ptr = o.ptr; od.elem = dtype_size(o.dtype); od.mn_major = false; od.inner = j.N; od.rows = j.M; od.row_stride = o.ld;
        for (int i = 0; i < 3; ++i) { od.bsz[i] = j.bsz[i]; od.bstride[i] = o.bstride[i]; }
        if ((uint64_t(j.N) * od.elem) % 16 == 0 && tma_compatible(od) && encode_tiled(c, &p.tm_out, od, kRowBytes / od.elem, 32, od.elem == 2 ? 2 : 0) == 0) p.tma_store = 1;
    }

    const unsigned grid = unsigned(std::min<uint64_t>(tiles * split, uint64_t(c->sm_count)));
    int rc;
    if (use_pair) {
        const uint64_t pair_tiles = launch_pairs;
        rc = launch_status(c, launch_gemm_pair(launch_env(c), j.kind, two_groups ? 2 : 1, p, pair_tiles));
    } else {
        rc = launch_status(c, launch_gemm_single(launch_env(c), j.kind, block_n, p, grid));
    }
    TRY(rc);
    if (peer) return run_peer_exchange(c, peer, static_cast<const float*>(ws), split, uint64_t(j.M) * j.N, o.scale, static_cast<float*>(o.ptr));
    if (split > 1) {
        ReduceOut r;
        memset(&r, 0, sizeof r);
        r.out = o.ptr; r.out_dtype = o.dtype; r.has_cast = o.has_cast; r.out_ld = o.ld;
        for (int i = 0; i < 3; ++i) { r.out_bstride[i] = o.bstride[i]; r.bsz[i] = j.bsz[i]; }
        r.M = j.M; r.N = j.N; r.batches = p.batches; r.splits = split; r.scale = o.scale; r.cast = o.cast;
        r.rng_philox = o.philox; r.seed = o.seed; r.offset = o.offset;
        r.pred = j.pred; r.pred_nonzero = j.pred_nonzero;
        const uint64_t total = uint64_t(j.M) * j.N * p.batches;
        const bool vec4 = j.N % 4 == 0 && o.ld % 4 == 0 && o.bstride[0] % 4 == 0 && o.bstride[1] % 4 == 0 && o.bstride[2] % 4 == 0 &&
                          (reinterpret_cast<uintptr_t>(o.ptr) & 15) == 0;
        if (vec4) splitk_reduce_vec4_kernel<<<grid_for(total / 4, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<const float*>(ws), r);
        else splitk_reduce_kernel<<<grid_for(total, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<const float*>(ws), r);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
    }
    return 0;
}

// ------------------------------------------------------------------------------------------ operand preparation
// Logical operand: element (mn, k) of batch (b0,b1,b2) at ptr[b . bstride + mn*mn_stride + k*k_stride].
struct LogicalOperand {
    const void* ptr;
    int dtype, bias, mode;
    uint64_t mn, k, mn_stride, k_stride;
    uint32_t bsz[3];
    uint64_t bstride[3];
};

enum PrepKind { PREP_NATIVE, PREP_FP8_TO_BF16, PREP_TF32_ROUND, PREP_SPLIT_A, PREP_SPLIT_B };

static int repack(mmeb200_ctx* c, const LogicalOperand& in, PrepKind kind, TmaOperand* out, uint64_t* k_out, const uint32_t* pred = nullptr,
                  uint32_t pred_nonzero = 0) {
    RepackParams r;
    memset(&r, 0, sizeof r);
    r.pred = pred; r.pred_nonzero = pred_nonzero;
    const int src_elem = dtype_size(in.dtype);
    int dst_elem = src_elem;
    uint64_t segs = 1;
    r.mode = 0;
    if (kind == PREP_FP8_TO_BF16) { r.mode = 1; dst_elem = 2; }
    else if (kind == PREP_TF32_ROUND) r.mode = 2;
    else if (kind == PREP_SPLIT_A) { r.mode = 3; segs = 3; }
    else if (kind == PREP_SPLIT_B) { r.mode = 4; segs = 3; }
    const uint64_t block_k = kRowBytes / dst_elem;
    const uint64_t seg = (segs == 1) ? in.k : ((in.k + block_k - 1) / block_k) * block_k;
    const uint64_t align = 16 / dst_elem;
    const uint64_t batches = uint64_t(in.bsz[0]) * in.bsz[1] * in.bsz[2];
    // Operands with a contiguous dimension keep their orientation and are converted four elements at a time
    // (repack_vec4_kernel); anything else is gathered element by element into a K-major copy.
    {
        const bool k_contig = in.k_stride == 1, mn_contig = in.mn_stride == 1 && !k_contig;
        const uint64_t C_ = k_contig ? in.k : in.mn, R_ = k_contig ? in.mn : in.k, rs = k_contig ? in.mn_stride : in.k_stride;
        bool ok = (k_contig || mn_contig) && C_ % 4 == 0 && rs % 4 == 0 && (reinterpret_cast<uintptr_t>(in.ptr) % (4 * src_elem)) == 0 && R_ && C_;
        if (mn_contig && src_elem == 4) ok = false;   // 32-bit operands must reach the tensor cores K-major: transposed below
        for (int i = 0; i < 3; ++i) ok = ok && (in.bsz[i] == 1 || in.bstride[i] % 4 == 0);
        if (ok) {
            RepackVecParams v;
            memset(&v, 0, sizeof v);
            v.pred = pred; v.pred_nonzero = pred_nonzero;
            const uint64_t c_ext = k_contig ? seg * segs : C_;
            const uint64_t ld = ((c_ext + align - 1) / align) * align;
            const uint64_t rows_out = k_contig ? R_ : seg * segs;
            void* dst = nullptr;
            const size_t bytes = size_t(batches) * rows_out * ld * dst_elem;
            TRY(arena_alloc(c, &dst, bytes));
            if (seg != in.k || ld != c_ext) CUDA_OK(c, cudaMemsetAsync(dst, 0, bytes, c->stream));   // padding reads as zeros
            v.src = in.ptr; v.dst = dst; v.R = R_; v.C = C_; v.r_stride = rs;
            for (int i = 0; i < 3; ++i) { v.bstride[i] = in.bstride[i]; v.bsz[i] = in.bsz[i]; }
            v.dst_ld = ld; v.dst_batch = rows_out * ld; v.seg = seg; v.seg_along_c = k_contig ? 1 : 0;
            v.mode = r.mode; v.src_elem = src_elem; v.dtype = in.dtype; v.bias = in.bias; v.inf_nan = in.mode;
            repack_vec4_kernel<<<grid_for(batches * R_ * (C_ / 4), 256, c->sm_count), 256, 0, c->stream>>>(v);
            c->launches++;
            CUDA_OK(c, cudaGetLastError());
            out->ptr = dst; out->elem = dst_elem; out->mn_major = !k_contig;
            out->inner = k_contig ? seg * segs : in.mn;
            out->rows = rows_out; out->row_stride = ld;
            uint64_t bs = v.dst_batch;
            for (int i = 0; i < 3; ++i) { out->bsz[i] = in.bsz[i]; out->bstride[i] = bs; bs *= in.bsz[i]; }
            *k_out = seg * segs;
            return 0;
        }
    }
    const uint64_t ld = ((seg * segs + align - 1) / align) * align;
    void* dst = nullptr;
    const size_t bytes = size_t(batches) * in.mn * ld * dst_elem;
    TRY(arena_alloc(c, &dst, bytes));
    if (segs > 1 || ld != in.k) CUDA_OK(c, cudaMemsetAsync(dst, 0, bytes, c->stream));
    if (src_elem == 4 && r.mode >= 2 && in.mn_stride == 1 && in.k_stride != 1 && in.mn && in.k) {
        // fp32 / tf32 with M or N contiguous: tiled transpose into the K-major copy (repack_transpose_f32_kernel)
        RepackTransposeParams t;
        memset(&t, 0, sizeof t);
        t.src = static_cast<const uint32_t*>(in.ptr); t.dst = static_cast<uint32_t*>(dst);
        t.mn = in.mn; t.k = in.k; t.k_stride = in.k_stride;
        for (int i = 0; i < 3; ++i) { t.bstride[i] = in.bstride[i]; t.bsz[i] = in.bsz[i]; }
        t.dst_ld = ld; t.seg = seg; t.mode = r.mode;
        const uint64_t tiles = ((in.mn + 31) / 32) * ((in.k + 31) / 32) * batches;
        repack_transpose_f32_kernel<<<unsigned(std::min<uint64_t>(tiles, uint64_t(c->sm_count) * 32)), 256, 0, c->stream>>>(t);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
        out->ptr = dst; out->elem = dst_elem; out->mn_major = false; out->inner = seg * segs; out->rows = in.mn; out->row_stride = ld;
        uint64_t bs2 = in.mn * ld;
        for (int i = 0; i < 3; ++i) { out->bsz[i] = in.bsz[i]; out->bstride[i] = bs2; bs2 *= in.bsz[i]; }
        *k_out = seg * segs;
        return 0;
    }
    r.src = in.ptr; r.dst = dst; r.rows = in.mn; r.k = in.k; r.row_stride = in.mn_stride; r.k_stride = in.k_stride;
    for (int i = 0; i < 3; ++i) { r.bstride[i] = in.bstride[i]; r.bsz[i] = in.bsz[i]; }
    r.dst_ld = ld; r.seg = seg; r.src_elem = src_elem; r.dtype = in.dtype; r.bias = in.bias; r.inf_nan = in.mode;
    const uint64_t total = batches * in.mn * in.k;
    if (total) {
        repack_kernel<<<grid_for(total, 256, c->sm_count), 256, 0, c->stream>>>(r);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
    }
    out->ptr = dst; out->elem = dst_elem; out->mn_major = false; out->inner = seg * segs; out->rows = in.mn; out->row_stride = ld;
    uint64_t bs = in.mn * ld;
    for (int i = 0; i < 3; ++i) { out->bsz[i] = in.bsz[i]; out->bstride[i] = bs; bs *= in.bsz[i]; }
    *k_out = seg * segs;
    return 0;
}

static int native_operand(const LogicalOperand& in, TmaOperand* out) {
    out->ptr = in.ptr;
    out->elem = dtype_size(in.dtype);
    const bool k_major = in.k_stride == 1;
    if (!k_major && in.mn_stride != 1) return -1;
    out->mn_major = !k_major;
    out->inner = k_major ? in.k : in.mn;
    out->rows = k_major ? in.mn : in.k;
    out->row_stride = k_major ? in.mn_stride : in.k_stride;
    for (int i = 0; i < 3; ++i) { out->bsz[i] = in.bsz[i]; out->bstride[i] = in.bstride[i]; }
    return 0;
}

// Can any code of this fp8 tensor mean something else to the reference than to the tensor cores? The tensor cores read
// 1-4-3 in the 'minimal' Inf/NaN convention and 1-5-2 in the 'full' one.
static bool fp8_may_hold_foreign_codes(const LogicalOperand& in) {
    const int ew = in.dtype == DT_FP8_143 ? 4 : 5;
    return !((ew == 4 && in.mode == 2) || (ew == 5 && in.mode == 0));
}
// Sets *flag (device memory, zeroed by the caller) when the tensor holds such a code. Stays on the stream: no host round trip.
static int fp8_scan_foreign_codes(mmeb200_ctx* c, const LogicalOperand& in, const mmeb200_tensor* whole, uint32_t* flag) {
    const uint64_t n = span_elems(whole);
    if (n == 0) return 0;
    fp8_scan_kernel<<<grid_for(n, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<const uint8_t*>(whole->data), n, in.dtype == DT_FP8_143 ? 4 : 5,
                                                                         in.mode, flag);
    c->launches++;
    CUDA_OK(c, cudaGetLastError());
    return 0;
}

// Decide the tensor-core kind for a dtype pair and turn both logical operands into TMA operands.
// fp8 operands whose convention the tensor cores may not share get TWO forms: `j` multiplies the codes natively and runs
// only if a device-side scan found no foreign code; `alt` (then *has_alt) decodes both operands exactly to bf16 first and
// runs only if the scan found one. Both are enqueued; the flag the scan leaves in device memory decides.
static int prepare_pair(mmeb200_ctx* c, const LogicalOperand& la, const LogicalOperand& lb, const mmeb200_tensor* ta,
                        const mmeb200_tensor* tb, GemmJob* j, float* scale, GemmJob* alt, float* alt_scale, bool* has_alt) {
    *scale = 1.0f;
    *alt_scale = 1.0f;
    *has_alt = false;
    const bool a8 = dtype_is_fp8(la.dtype), b8 = dtype_is_fp8(lb.dtype);
    if (a8 != b8 || (!a8 && la.dtype != lb.dtype))
        return c->fail(MMEB200_ERR_UNSUPPORTED, "operand data types %d and %d cannot be mixed", la.dtype, lb.dtype);
    uint64_t ka = la.k, kb = lb.k;
    if (la.dtype == DT_BF16) {
        j->kind = KIND_F16;
        if (native_operand(la, &j->a) != 0 || !tma_compatible(j->a)) TRY(repack(c, la, PREP_NATIVE, &j->a, &ka));
        if (native_operand(lb, &j->b) != 0 || !tma_compatible(j->b)) TRY(repack(c, lb, PREP_NATIVE, &j->b, &kb));
        j->a.hw_fmt = j->b.hw_fmt = 1;
    } else if (a8) {
        const bool may_a = fp8_may_hold_foreign_codes(la), may_b = fp8_may_hold_foreign_codes(lb);
        uint32_t* flag = nullptr;
        if (may_a || may_b) {
            TRY(arena_alloc(c, reinterpret_cast<void**>(&flag), 4));
            CUDA_OK(c, cudaMemsetAsync(flag, 0, 4, c->stream));
            if (may_a) TRY(fp8_scan_foreign_codes(c, la, ta, flag));
            if (may_b) TRY(fp8_scan_foreign_codes(c, lb, tb, flag));
            // some code may mean Inf / NaN / another number to the reference than to the tensor cores: the form that decodes
            // both operands exactly to bf16 on the device and multiplies those runs if the scan raised the flag
            *alt = *j;
            alt->kind = KIND_F16;
            alt->pred = flag; alt->pred_nonzero = 1;
            uint64_t kda = la.k, kdb = lb.k;
            TRY(repack(c, la, PREP_FP8_TO_BF16, &alt->a, &kda, flag, 1));
            TRY(repack(c, lb, PREP_FP8_TO_BF16, &alt->b, &kdb, flag, 1));
            alt->a.hw_fmt = alt->b.hw_fmt = 1;
            alt->K = uint32_t(std::max(kda, kdb));
            *has_alt = true;
            j->pred = flag; j->pred_nonzero = 0;
        }
        j->kind = KIND_F8;
        if (native_operand(la, &j->a) != 0 || !tma_compatible(j->a)) TRY(repack(c, la, PREP_NATIVE, &j->a, &ka, j->pred, 0));
        if (native_operand(lb, &j->b) != 0 || !tma_compatible(j->b)) TRY(repack(c, lb, PREP_NATIVE, &j->b, &kb, j->pred, 0));
        j->a.hw_fmt = la.dtype == DT_FP8_143 ? 0 : 1;
        j->b.hw_fmt = lb.dtype == DT_FP8_143 ? 0 : 1;
        // the tensor cores decode 1-4-3 with bias 7 and 1-5-2 with bias 15: fold the difference
        const int ea = (la.dtype == DT_FP8_143 ? 7 : 15) - la.bias;
        const int eb = (lb.dtype == DT_FP8_143 ? 7 : 15) - lb.bias;
        *scale = ldexpf(1.0f, ea + eb);
    } else if (la.dtype == DT_TF32) {
        j->kind = KIND_TF32;
        TRY(repack(c, la, PREP_TF32_ROUND, &j->a, &ka));
        TRY(repack(c, lb, PREP_TF32_ROUND, &j->b, &kb));
        j->a.hw_fmt = j->b.hw_fmt = 2;
    } else {  // fp32 / fp32_ieee: three tf32 products per element pair
        j->kind = KIND_TF32;
        TRY(repack(c, la, PREP_SPLIT_A, &j->a, &ka));
        TRY(repack(c, lb, PREP_SPLIT_B, &j->b, &kb));
        j->a.hw_fmt = j->b.hw_fmt = 2;
    }
    j->K = uint32_t(std::max(ka, kb));
    return 0;
}

static int make_cast_spec(mmeb200_ctx* c, const mmeb200_tensor* out, const mmeb200_cast_params* cp, CastSpec* s) {
    memset(s, 0, sizeof *s);
    s->out_dtype = out->dtype == DT_FP32_IEEE ? DT_FP32 : out->dtype;
    if (s->out_dtype == DT_TF32) return c->fail(MMEB200_ERR_UNSUPPORTED, "tf32 is not an output data type");
    s->exp_width = out->dtype == DT_FP8_143 ? 4 : 5;
    s->bias = int(out->fp_bias);
    s->mode = out->inf_nan_mode;
    if (cp) {
        s->rm = cp->rounding; s->relu = cp->relu; s->clip = cp->clip_fp; s->clip_inf_in = cp->clip_inf_in;
        s->ftz = cp->flush_denorms; s->sftz = cp->stochastic_ftz_fp8;
        if (!(s->rm >= 0 && s->rm <= 7 && s->rm != 5)) return c->fail(MMEB200_ERR_INVALID_ARG, "rounding mode %d is not valid", s->rm);
    }
    return 0;
}

// ------------------------------------------------------------------------------------------ LFSR support
static uint32_t gf2_apply_host(const uint32_t* cols, uint32_t s) {
    uint32_t r = 0;
    for (int b = 0; b < 32; ++b)
        if ((s >> b) & 1u) r ^= cols[b];
    return r;
}
static int ensure_jump_table(mmeb200_ctx* c) {
    if (c->d_jump && c->jump_poly == c->polynomial && !c->h_jump.empty()) return 0;
    c->h_jump.assign(32 * 32, 0);
    for (int b = 0; b < 32; ++b) c->h_jump[b] = lfsr32_step(1u << b, c->polynomial);
    for (int j = 1; j < 32; ++j)
        for (int b = 0; b < 32; ++b) c->h_jump[32 * j + b] = gf2_apply_host(&c->h_jump[32 * (j - 1)], c->h_jump[32 * (j - 1) + b]);
    if (!c->d_jump) CUDA_OK(c, cudaMalloc(&c->d_jump, 32 * 32 * 4));
    CUDA_OK(c, cudaMemcpyAsync(c->d_jump, c->h_jump.data(), 32 * 32 * 4, cudaMemcpyHostToDevice, c->stream));
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    c->jump_poly = c->polynomial;
    return 0;
}
static uint32_t lfsr_jump_host(mmeb200_ctx* c, uint32_t s, uint64_t steps) {
    for (int j = 0; steps; ++j, steps >>= 1)
        if (steps & 1) s = gf2_apply_host(&c->h_jump[32 * j], s);
    return s;
}

// fp32 accumulator -> out, on device pointers. Dense tensors only (as the reference requires).
static int run_cast(mmeb200_ctx* c, void* out, uint32_t* acc, uint64_t n, const CastSpec& s, const mmeb200_cast_params* cp) {
    if (n == 0) return 0;
    const bool random = cast_needs_random(s);
    const int rng = cp ? cp->rng_kind : MMEB200_RNG_LFSR;
    const bool use_lfsr = random && rng != MMEB200_RNG_PHILOX && s.out_dtype != DT_FP32;
    if (!use_lfsr) {
        const bool philox = random && rng == MMEB200_RNG_PHILOX;
        const uint64_t offset = cp ? cp->rng_offset : 0;
        CastTier tier;
        memset(&tier, 0, sizeof tier);
        tier.kind = CAST_GENERAL;
        if (s.out_dtype == DT_BF16 && s.rm == RM_NE && !s.clip && !s.ftz && !s.clip_inf_in) tier.kind = CAST_BF16_RNE;
        else if (cast_is_fp8_hw(s)) {
            tier.kind = CAST_FP8_HW;
            tier.hw = fp8_hw_cast(s);
        } else if (philox && s.rm == RM_SR && (offset & 7u) == 0 && !s.ftz && (s.out_dtype == DT_BF16 || (dtype_is_fp8(s.out_dtype) && !s.sftz)))
            tier.kind = CAST_SR8;
        else if ((!philox || (offset & 3u) == 0) && (s.out_dtype == DT_BF16 || (dtype_is_fp8(s.out_dtype) && !s.ftz && !s.sftz)))
            tier.kind = CAST_FLAT;
        cast_kernel<<<grid_for((n + 15) / 16, 256, c->sm_count), 256, 0, c->stream>>>(out, acc, n, s, philox ? 1 : 0, cp ? cp->rng_seed : 0, offset, tier);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
        return 0;
    }
    // the reference's LFSR stream
    const uint32_t lanes = (s.out_dtype == DT_BF16) ? 64 : 128;
    if (c->lfsr.size() < lanes) return c->fail(MMEB200_ERR_INVALID_ARG, "need %u LFSR registers, context has %zu", lanes, c->lfsr.size());
    TRY(ensure_jump_table(c));
    if (!c->d_lfsr) CUDA_OK(c, cudaMalloc(&c->d_lfsr, 128 * 4));
    CUDA_OK(c, cudaMemcpyAsync(c->d_lfsr, c->lfsr.data(), lanes * 4, cudaMemcpyHostToDevice, c->stream));
    const uint32_t spt = 64;
    const uint64_t steps = (n + lanes - 1) / lanes;
    const uint64_t chunks = (steps + spt - 1) / spt;
    const uint64_t threads = chunks * lanes;
    cast_lfsr_kernel<<<unsigned((threads + 127) / 128), 128, 0, c->stream>>>(out, acc, n, s, c->d_lfsr, c->d_jump, c->polynomial, lanes,
                                                                            spt, chunks);
    c->launches++;
    CUDA_OK(c, cudaGetLastError());
    if (random) {  // advance the context's registers like m_lfsr in the reference
        CUDA_OK(c, cudaStreamSynchronize(c->stream));  // d_lfsr upload must finish before the host copy changes
        for (uint32_t r = 0; r < lanes && r < n; ++r) {
            const uint64_t uses = (n - r + lanes - 1) / lanes;
            c->lfsr[r] = lfsr_jump_host(c, c->lfsr[r], uses);
        }
    }
    return 0;
}

// The device-side part of doBatchGemm: all three descriptors point at device memory.
// rng_extra_offset shifts the Philox counter when the caller runs a row block of a larger product;
// row blocks also keep the reduction unsplit, so that every row sees the same summation order as in
// a single launch.
// Bit-exact Gaudi3 accumulation (MMEB200_ACC_CHIP_EXACT): out[b][m][n] (fp32) = sum over k in the reference's block order.
static int run_exact_gemm(mmeb200_ctx* c, const LogicalOperand& la, const LogicalOperand& lb, uint64_t M, uint64_t N, void* out,
                          uint64_t out_ld, const uint32_t bsz[3], const uint64_t out_bstride[3]) {
    if (c->chip != MMEB200_CHIP_GAUDI3)
        return c->fail(MMEB200_ERR_UNSUPPORTED, "bit-exact accumulation is implemented for the Gaudi3 model only");
    auto narrow = [](int dt) { return dt == DT_BF16 || dt == DT_FP8_143 || dt == DT_FP8_152; };
    const bool wide = (la.dtype == DT_FP32 || la.dtype == DT_TF32) && lb.dtype == la.dtype;
    if (!wide && (!narrow(la.dtype) || !narrow(lb.dtype) || (la.dtype == DT_BF16) != (lb.dtype == DT_BF16)))
        return c->fail(MMEB200_ERR_UNSUPPORTED, "bit-exact accumulation takes bf16 x bf16, fp8 x fp8, fp32 x fp32 or tf32 x tf32 operands");
    ExactGemmParams e;
    memset(&e, 0, sizeof e);
    e.a = la.ptr; e.b = lb.ptr; e.out = static_cast<float*>(out);
    e.M = uint32_t(M); e.N = uint32_t(N); e.K = uint32_t(la.k);
    e.a_mn_stride = la.mn_stride; e.a_k_stride = la.k_stride; e.b_mn_stride = lb.mn_stride; e.b_k_stride = lb.k_stride;
    for (int i = 0; i < 3; ++i) {
        e.bsz[i] = bsz[i];
        e.a_bstride[i] = la.bsz[i] == 1 ? 0 : la.bstride[i];   // size-1 batch dims broadcast
        e.b_bstride[i] = lb.bsz[i] == 1 ? 0 : lb.bstride[i];
        e.out_bstride[i] = out_bstride[i];
    }
    e.out_ld = out_ld;
    e.a_dtype = la.dtype; e.a_bias = la.bias; e.a_mode = la.mode;
    e.b_dtype = lb.dtype; e.b_bias = lb.bias; e.b_mode = lb.mode;
    const uint64_t edge = wide ? 16 : kExactTile;
    const uint64_t tiles = ((M + edge - 1) / edge) * ((N + edge - 1) / edge) * bsz[0] * bsz[1] * bsz[2];
    if (tiles == 0) return 0;
    const unsigned grid = unsigned(std::min<uint64_t>(tiles, uint64_t(c->sm_count) * 8));
    if (wide) gaudi3_exact_gemm_wide_kernel<<<grid, 256, 0, c->stream>>>(e);
    else gaudi3_exact_gemm_kernel<<<grid, 256, 0, c->stream>>>(e);
    c->launches++;
    CUDA_OK(c, cudaGetLastError());
    return 0;
}

static int bgemm_core(mmeb200_ctx* c, const mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w, int op,
                      const mmeb200_cast_params* cast, uint64_t rng_extra_offset, bool row_block = false) {
    const bool tA = (op == MMEB200_OP_ATB || op == MMEB200_OP_ATBT), tB = (op == MMEB200_OP_ABT || op == MMEB200_OP_ATBT);
    const uint64_t M = tA ? x->sizes[0] : x->sizes[1], K = tA ? x->sizes[1] : x->sizes[0];
    const uint64_t N = tB ? w->sizes[1] : w->sizes[0];
    LogicalOperand la, lb;
    la.ptr = x->data; la.dtype = x->dtype; la.bias = int(x->fp_bias); la.mode = x->inf_nan_mode;
    la.mn = M; la.k = K;
    la.mn_stride = tA ? 1 : x->strides[1];
    la.k_stride = tA ? x->strides[1] : 1;
    lb.ptr = w->data; lb.dtype = w->dtype; lb.bias = int(w->fp_bias); lb.mode = w->inf_nan_mode;
    lb.mn = N; lb.k = K;
    lb.mn_stride = tB ? w->strides[1] : 1;
    lb.k_stride = tB ? 1 : w->strides[1];
    for (int i = 0; i < 3; ++i) {
        la.bsz[i] = x->sizes[2 + i]; la.bstride[i] = x->strides[2 + i];
        lb.bsz[i] = w->sizes[2 + i]; lb.bstride[i] = w->strides[2 + i];
    }
    if (c->acc_mode == MMEB200_ACC_CHIP_EXACT) {
        const uint32_t bsz[3] = {out->sizes[2], out->sizes[3], out->sizes[4]};
        if (K == 0) return c->fail(MMEB200_ERR_INVALID_ARG, "empty common dimension");
        if (!cast) {
            const uint64_t obs[3] = {out->strides[2], out->strides[3], out->strides[4]};
            return run_exact_gemm(c, la, lb, M, N, out->data, out->strides[1], bsz, obs);
        }
        if (!is_dense(out)) return c->fail(MMEB200_ERR_UNSUPPORTED, "a cast after bit-exact accumulation needs a dense output tensor");
        CastSpec ecs;
        TRY(make_cast_spec(c, out, cast, &ecs));
        void* acc = nullptr;
        const uint64_t n = num_elems(out);
        TRY(arena_alloc(c, &acc, n * 4));
        uint64_t obs[3], bs = M * N;
        for (int i = 0; i < 3; ++i) { obs[i] = bs; bs *= out->sizes[2 + i]; }
        TRY(run_exact_gemm(c, la, lb, M, N, acc, N, bsz, obs));
        return run_cast(c, out->data, static_cast<uint32_t*>(acc), n, ecs, cast);
    }
    GemmJob job, alt;
    float scale = 1.0f, alt_scale = 1.0f;
    bool has_alt = false;
    TRY(prepare_pair(c, la, lb, x, w, &job, &scale, &alt, &alt_scale, &has_alt));
    for (GemmJob* g : {&job, &alt}) {
        g->M = uint32_t(M); g->N = uint32_t(N);
        if (row_block) g->force_split = 1;
        for (int i = 0; i < 3; ++i) g->bsz[i] = out->sizes[2 + i];
    }

    OutSpec o;
    memset(&o, 0, sizeof o);
    o.ld = out->strides[1];
    for (int i = 0; i < 3; ++i) { o.bsz[i] = out->sizes[2 + i]; o.bstride[i] = out->strides[2 + i]; }
    CastSpec cs;
    TRY(make_cast_spec(c, out, cast, &cs));
    const bool random = cast && cast_needs_random(cs);
    const bool fuse = !cast || !random || cast->rng_kind == MMEB200_RNG_PHILOX || cs.out_dtype == DT_FP32;
    // both forms of an fp8 GEMM whose operands' convention differs from the tensor cores' are enqueued; the device runs one
    auto run_forms = [&]() -> int {
        o.scale = scale;
        TRY(run_gemm(c, job, o));
        if (has_alt) {
            o.scale = alt_scale;
            TRY(run_gemm(c, alt, o));
        }
        return 0;
    };
    if (fuse) {
        o.ptr = out->data; o.dtype = cs.out_dtype; o.has_cast = cast != nullptr; o.cast = cs;
        o.philox = random && cast->rng_kind == MMEB200_RNG_PHILOX;
        o.seed = cast ? cast->rng_seed : 0; o.offset = (cast ? cast->rng_offset : 0) + rng_extra_offset;
        TRY(run_forms());
    } else {
        // LFSR-ordered stochastic rounding needs the reference's sequential element order:
        // accumulate to fp32 scratch, then run the standalone cast
        if (!is_dense(out)) return c->fail(MMEB200_ERR_UNSUPPORTED, "LFSR stochastic rounding needs a dense output tensor");
        void* acc = nullptr;
        const uint64_t n = num_elems(out);
        TRY(arena_alloc(c, &acc, n * 4));
        o.ptr = acc; o.dtype = DT_FP32; o.has_cast = false; o.ld = N;
        uint64_t bs = M * N;
        for (int i = 0; i < 3; ++i) { o.bstride[i] = bs; bs *= out->sizes[2 + i]; }
        TRY(run_forms());
        TRY(run_cast(c, out->data, static_cast<uint32_t*>(acc), n, cs, cast));
    }
    return 0;
}


// Host-tensor GEMMs large enough for the PCIe copies to dominate are run as a pipeline: B is
// uploaded once, then A arrives in row blocks; block i is multiplied while block i+1 uploads and
// block i-1's output downloads (PCIe is full duplex, the copies of the two directions overlap).
static bool host_pipeline_applies(const mmeb200_ctx* c, const mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w, int op,
                                  const mmeb200_cast_params* cast, uint64_t M, uint64_t N, uint64_t K) {
    if (c->tune.host_pipeline == 0) return false;
    // x and the output stream through in row blocks; w is uploaded once, or is already resident (a multi-GPU driver that
    // spread it over NVLink)
    if (out->mem_space != MMEB200_MEM_HOST || x->mem_space != MMEB200_MEM_HOST) return false;
    if (op != MMEB200_OP_AB && op != MMEB200_OP_ABT) return false;  // rows of x must be rows of the product
    for (int d = 2; d < 5; ++d)
        if (out->sizes[d] != 1 || x->sizes[d] != 1 || w->sizes[d] != 1) return false;
    if (!is_dense(out) || !is_dense(x) || !is_dense(w)) return false;
    const bool bf = x->dtype == DT_BF16 && w->dtype == DT_BF16;
    auto native8 = [](const mmeb200_tensor* t) { return (t->dtype == DT_FP8_143 && t->inf_nan_mode == 2) || (t->dtype == DT_FP8_152 && t->inf_nan_mode == 0); };
    if (!bf && !(native8(x) && native8(w))) return false;  // other formats scan or convert whole tensors first
    if (cast) {
        CastSpec cs;
        memset(&cs, 0, sizeof cs);
        cs.rm = cast->rounding; cs.sftz = cast->stochastic_ftz_fp8;
        if (cast_needs_random(cs) && cast->rng_kind != MMEB200_RNG_PHILOX) return false;  // LFSR order is sequential over the whole tensor
    } else if (out->dtype != DT_FP32 && out->dtype != DT_FP32_IEEE) return false;
    const uint64_t e = dtype_size(x->dtype);
    if ((K * e) % 16 || (reinterpret_cast<uintptr_t>(x->data) & 15)) return false;
    const uint64_t bytes = M * K * e + K * N * e + M * N * dtype_size(out->dtype);
    return M >= 512 && bytes >= (uint64_t(32) << 20);
}

static int bgemm_host_pipelined(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w, int op,
                                const mmeb200_cast_params* cast, uint64_t M, uint64_t N, uint64_t K) {
    constexpr int kMaxChunks = 16;
    if (!c->s_h2d) {
        CUDA_OK(c, cudaStreamCreateWithFlags(&c->s_h2d, cudaStreamNonBlocking));
        CUDA_OK(c, cudaStreamCreateWithFlags(&c->s_d2h, cudaStreamNonBlocking));
        for (int i = 0; i < kMaxChunks + 1; ++i) {
            CUDA_OK(c, cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming));
            CUDA_OK(c, cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming));
        }
    }
    const uint64_t e = dtype_size(x->dtype), eo = dtype_size(out->dtype);
    uint8_t *dA = nullptr, *dB = nullptr, *dO = nullptr;
    const bool w_resident = w->mem_space == MMEB200_MEM_DEVICE;
    TRY(arena_alloc(c, reinterpret_cast<void**>(&dA), M * K * e));
    if (!w_resident) TRY(arena_alloc(c, reinterpret_cast<void**>(&dB), K * N * e));
    TRY(arena_alloc(c, reinterpret_cast<void**>(&dO), M * N * eo));
    // the arena may still be read by earlier work of this context's stream
    CUDA_OK(c, cudaEventRecord(c->ev_in[kMaxChunks], c->stream));
    CUDA_OK(c, cudaStreamWaitEvent(c->s_h2d, c->ev_in[kMaxChunks], 0));
    CUDA_OK(c, cudaStreamWaitEvent(c->s_d2h, c->ev_in[kMaxChunks], 0));
    if (!w_resident) CUDA_OK(c, cudaMemcpyAsync(dB, w->data, K * N * e, cudaMemcpyHostToDevice, c->s_h2d));
    // row blocks: multiples of the 128-row tile, about 8 of them
    uint64_t rows_per = ((M + 7) / 8 + 127) / 128 * 128;
    int nch = int((M + rows_per - 1) / rows_per);
    if (nch > kMaxChunks) { rows_per = ((M + kMaxChunks - 1) / kMaxChunks + 127) / 128 * 128; nch = int((M + rows_per - 1) / rows_per); }
    mmeb200_tensor tw = *w;
    if (!w_resident) { tw.data = dB; tw.mem_space = MMEB200_MEM_DEVICE; }
    for (int i = 0; i < nch; ++i) {
        const uint64_t r0 = uint64_t(i) * rows_per, rows = std::min<uint64_t>(rows_per, M - r0);
        CUDA_OK(c, cudaMemcpyAsync(dA + r0 * K * e, static_cast<const uint8_t*>(x->data) + r0 * K * e, rows * K * e, cudaMemcpyHostToDevice, c->s_h2d));
        CUDA_OK(c, cudaEventRecord(c->ev_in[i], c->s_h2d));
        CUDA_OK(c, cudaStreamWaitEvent(c->stream, c->ev_in[i], 0));
        mmeb200_tensor tx = *x, to = *out;
        tx.data = dA + r0 * K * e; tx.mem_space = MMEB200_MEM_DEVICE; tx.sizes[1] = uint32_t(rows);
        to.data = dO + r0 * N * eo; to.mem_space = MMEB200_MEM_DEVICE; to.sizes[1] = uint32_t(rows);
        TRY(bgemm_core(c, &to, &tx, &tw, op, cast, r0 * N, true));
        CUDA_OK(c, cudaEventRecord(c->ev_done[i], c->stream));
        CUDA_OK(c, cudaStreamWaitEvent(c->s_d2h, c->ev_done[i], 0));
        CUDA_OK(c, cudaMemcpyAsync(static_cast<uint8_t*>(out->data) + r0 * N * eo, dO + r0 * N * eo, rows * N * eo, cudaMemcpyDeviceToHost, c->s_d2h));
    }
    CUDA_OK(c, cudaStreamSynchronize(c->s_d2h));
    return finish_call(c, true);
}

// ------------------------------------------------------------------------------------------ C ABI: context
extern "C" {

const char* mmeb200_version(void) { return "mme_b200 0.1 sm_100a"; }

int mmeb200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int mmeb200_create(mmeb200_ctx** out_ctx, int chip, int device, unsigned seed, uint32_t lfsr_num_regs, const uint32_t* lfsr,
                   uint32_t polynomial) {
    if (!out_ctx) return MMEB200_ERR_INVALID_ARG;
    *out_ctx = nullptr;
    if (chip < 0 || chip > 2) return MMEB200_ERR_INVALID_ARG;
    int n = mmeb200_device_count();
    if (n <= 0) return MMEB200_ERR_NO_DEVICE;
    if (device < 0 || device >= n) return MMEB200_ERR_INVALID_ARG;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MMEB200_ERR_CUDA;
    if (prop.major != 10) return MMEB200_ERR_NO_DEVICE;  // kernels are built for sm_100a only
    if (cudaSetDevice(device) != cudaSuccess) return MMEB200_ERR_CUDA;
    mmeb200_ctx* c = new mmeb200_ctx();
    c->device = device; c->chip = chip; c->seed = seed; c->sm_count = prop.multiProcessorCount;
    c->tune.pair = env_int("MME_B200_PAIR", -1);
    c->tune.block_n = env_int("MME_B200_BLOCK_N", -1);
    c->tune.split_k = env_int("MME_B200_SPLIT_K", -1);
    c->tune.epi_groups = env_int("MME_B200_EPI_GROUPS", -1);
    c->tune.raster_gm = env_int("MME_B200_GM", -1);
    c->tune.tma_store = getenv("MME_B200_NO_TMA_STORE") ? 0 : -1;
    c->tune.host_pipeline = getenv("MME_B200_NO_HOST_PIPELINE") ? 0 : -1;
    c->tune.tile_n = env_int("MME_B200_TILE_N", -1);
    c->tune.stream_k = env_int("MME_B200_STREAM_K", -1);
    c->tune.dependent_launch = env_int("MME_B200_DEPENDENT_LAUNCH", -1);
    if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess || cudaMalloc(&c->d_status, 64) != cudaSuccess ||
        cudaMallocHost(&c->h_status, 64) != cudaSuccess || cudaEventCreate(&c->ev0) != cudaSuccess || cudaEventCreate(&c->ev1) != cudaSuccess) {
        delete c;
        return MMEB200_ERR_CUDA;
    }
    c->stream = c->own_stream;
    cudaMemsetAsync(c->d_status, 0, 64, c->stream);
    if (lfsr_num_regs == 0) lfsr_num_regs = 256;
    c->lfsr.resize(lfsr_num_regs);
    for (uint32_t i = 0; i < lfsr_num_regs; ++i) c->lfsr[i] = lfsr ? lfsr[i] : i + 2;
    if (polynomial == 0) {
        std::mt19937 gen(seed);
        std::uniform_int_distribution<> distr(25, 63);
        polynomial = uint32_t(distr(gen));
    }
    c->polynomial = polynomial;
    *out_ctx = c;
    return MMEB200_OK;
}

void mmeb200_destroy(mmeb200_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    if (c->s_side) {
        cudaStreamSynchronize(c->s_side);
        cudaStreamDestroy(c->s_side);
        cudaEventDestroy(c->ev_scatter);
        cudaEventDestroy(c->ev_gather);
    }
    for (auto& b : c->arena) cudaFree(b.ptr);
    if (c->aux) cudaFree(c->aux);
    if (c->sk_ws) cudaFree(c->sk_ws);
    if (c->sk_flags) cudaFree(c->sk_flags);
    if (c->d_status) cudaFree(c->d_status);
    if (c->h_status) cudaFreeHost(c->h_status);
    if (c->d_jump) cudaFree(c->d_jump);
    if (c->d_lfsr) cudaFree(c->d_lfsr);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    for (int i = 0; i < 17; ++i) {
        if (c->ev_in[i]) cudaEventDestroy(c->ev_in[i]);
        if (c->ev_done[i]) cudaEventDestroy(c->ev_done[i]);
    }
    if (c->s_h2d) cudaStreamDestroy(c->s_h2d);
    if (c->s_d2h) cudaStreamDestroy(c->s_d2h);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
}

int mmeb200_set_accumulation(mmeb200_ctx* c, int mode) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    if (mode != MMEB200_ACC_TENSOR_CORE && mode != MMEB200_ACC_CHIP_EXACT) return c->fail(MMEB200_ERR_INVALID_ARG, "accumulation mode %d is not valid", mode);
    if (mode == MMEB200_ACC_CHIP_EXACT && c->chip != MMEB200_CHIP_GAUDI3)
        return c->fail(MMEB200_ERR_UNSUPPORTED, "bit-exact accumulation is implemented for the Gaudi3 model only");
    c->acc_mode = mode;
    return 0;
}

int mmeb200_set_option(mmeb200_ctx* c, const char* name, int value) {
    if (!c || !name) return MMEB200_ERR_INVALID_ARG;
    struct { const char* name; int Tuning::*field; } const table[] = {
        {"pair", &Tuning::pair}, {"block_n", &Tuning::block_n}, {"split_k", &Tuning::split_k}, {"epi_groups", &Tuning::epi_groups},
        {"raster_gm", &Tuning::raster_gm}, {"tma_store", &Tuning::tma_store}, {"host_pipeline", &Tuning::host_pipeline},
        {"tile_n", &Tuning::tile_n}, {"stream_k", &Tuning::stream_k}, {"dependent_launch", &Tuning::dependent_launch}};
    for (const auto& t : table)
        if (strcmp(t.name, name) == 0) {
            c->tune.*(t.field) = value < 0 ? -1 : value;
            return 0;
        }
    return c->fail(MMEB200_ERR_INVALID_ARG, "unknown option '%s'", name);
}

int mmeb200_set_stream(mmeb200_ctx* c, void* s) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    c->stream = s ? static_cast<cudaStream_t>(s) : c->own_stream;
    return 0;
}
int mmeb200_limit_num_of_threads(mmeb200_ctx* c, unsigned) { return c ? 0 : MMEB200_ERR_INVALID_ARG; }
const char* mmeb200_last_error(const mmeb200_ctx* c) { return c ? c->err.c_str() : "null context"; }
uint64_t mmeb200_launch_count(const mmeb200_ctx* c) { return c ? c->launches : 0; }

int mmeb200_sync(mmeb200_ctx* c, uint64_t timeout_ns) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    if (timeout_ns) {
        CUDA_OK(c, cudaEventRecord(c->ev1, c->stream));
        const auto t0 = std::chrono::steady_clock::now();
        while (true) {
            cudaError_t q = cudaEventQuery(c->ev1);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady) return c->fail(MMEB200_ERR_CUDA, "cudaEventQuery: %s", cudaGetErrorString(q));
            const uint64_t el = std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
            if (el > timeout_ns) return c->fail(MMEB200_ERR_TIMEOUT, "work did not finish within %llu ns", (unsigned long long) timeout_ns);
        }
    }
    return collect_status(c);
}

int mmeb200_malloc(mmeb200_ctx* c, void** p, size_t bytes) {
    if (!c || !p) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaMalloc(p, bytes ? bytes : 16));
    return 0;
}
int mmeb200_free(mmeb200_ctx* c, void* p) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    CUDA_OK(c, cudaFree(p));
    return 0;
}
int mmeb200_memcpy_h2d(mmeb200_ctx* c, void* d, const void* h, size_t bytes) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, c->stream));
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    return 0;
}
int mmeb200_memcpy_d2h(mmeb200_ctx* c, void* h, const void* d, size_t bytes) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, c->stream));
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    return 0;
}
int mmeb200_memset(mmeb200_ctx* c, void* d, int value, size_t bytes) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaMemsetAsync(d, value, bytes, c->stream));
    return 0;
}
int mmeb200_mem_info(mmeb200_ctx* c, size_t* free_bytes, size_t* total_bytes) {
    if (!c || !free_bytes || !total_bytes) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaMemGetInfo(free_bytes, total_bytes));
    return 0;
}
int mmeb200_host_alloc(void** p, size_t bytes) {
    if (!p) return MMEB200_ERR_INVALID_ARG;
    return cudaMallocHost(p, bytes ? bytes : 16) == cudaSuccess ? 0 : MMEB200_ERR_CUDA;
}
int mmeb200_host_free(void* p) { return cudaFreeHost(p) == cudaSuccess ? 0 : MMEB200_ERR_CUDA; }

int mmeb200_timer_start(mmeb200_ctx* c) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    CUDA_OK(c, cudaEventRecord(c->ev0, c->stream));
    return 0;
}
int mmeb200_timer_stop(mmeb200_ctx* c, float* ms) {
    if (!c || !ms) return MMEB200_ERR_INVALID_ARG;
    if (c->gather_pending) {   // a deferred exchange output belongs to the timed work
        CUDA_OK(c, cudaStreamWaitEvent(c->stream, c->ev_gather, 0));
        c->gather_pending = false;
    }
    CUDA_OK(c, cudaEventRecord(c->ev1, c->stream));
    CUDA_OK(c, cudaEventSynchronize(c->ev1));
    CUDA_OK(c, cudaEventElapsedTime(ms, c->ev0, c->ev1));
    return 0;
}

int mmeb200_get_lfsr(mmeb200_ctx* c, uint32_t* regs, uint32_t n, uint32_t* poly) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    for (uint32_t i = 0; regs && i < n && i < c->lfsr.size(); ++i) regs[i] = c->lfsr[i];
    if (poly) *poly = c->polynomial;
    return 0;
}
int mmeb200_set_lfsr(mmeb200_ctx* c, const uint32_t* regs, uint32_t n, uint32_t poly) {
    if (!c || (n && !regs)) return MMEB200_ERR_INVALID_ARG;
    if (n) c->lfsr.assign(regs, regs + n);
    if (poly) c->polynomial = poly;
    return 0;
}

// ------------------------------------------------------------------------------------------ doBatchGemm
int mmeb200_bgemm(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w, int op,
                  const mmeb200_cast_params* cast) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    TRY(check_tensor(c, out, "output"));
    TRY(check_tensor(c, x, "x"));
    TRY(check_tensor(c, w, "w"));
    if (op < MMEB200_OP_AB || op > MMEB200_OP_ATBT) return c->fail(MMEB200_ERR_INVALID_ARG, "operation %d is not a batch-gemm operation", op);
    if (!cast && out->dtype != DT_FP32 && out->dtype != DT_FP32_IEEE)
        return c->fail(MMEB200_ERR_INVALID_ARG, "without cast parameters the output must be the fp32 accumulator");
    for (int d = 2; d < 5; ++d)
        if (!((x->sizes[d] == out->sizes[d] || x->sizes[d] == 1) && (w->sizes[d] == out->sizes[d] || w->sizes[d] == 1)))
            return c->fail(MMEB200_ERR_INVALID_ARG, "batch dims doesnt match !");
    const bool tA = (op == MMEB200_OP_ATB || op == MMEB200_OP_ATBT), tB = (op == MMEB200_OP_ABT || op == MMEB200_OP_ATBT);
    const uint64_t M = tA ? x->sizes[0] : x->sizes[1], K = tA ? x->sizes[1] : x->sizes[0];
    const uint64_t Kb = tB ? w->sizes[0] : w->sizes[1], N = tB ? w->sizes[1] : w->sizes[0];
    arena_reset(c);
    const bool any_host = out->mem_space == MMEB200_MEM_HOST || x->mem_space == MMEB200_MEM_HOST || w->mem_space == MMEB200_MEM_HOST;
    Staged so, sx, sw;
    // zero common dimension: the reference writes zeros (mme_reference_impl.cpp:204-216)
    if (num_elems(x) == 0 || num_elems(w) == 0) {
        if (num_elems(x) != num_elems(w)) return c->fail(MMEB200_ERR_INVALID_ARG, "One of the input tensors is zero-size, while the other is not");
        TRY(stage_in(c, out, &so, false));
        CUDA_OK(c, cudaMemsetAsync(so.t.data, 0, num_elems(out) * dtype_size(out->dtype), c->stream));
        so.bytes = num_elems(out) * dtype_size(out->dtype);
        TRY(stage_out(c, &so));
        return finish_call(c, any_host);
    }
    if (K != Kb) return c->fail(MMEB200_ERR_INVALID_ARG, "Common dim doesnt match between input A\\B");
    if (out->sizes[0] != N || out->sizes[1] != M) return c->fail(MMEB200_ERR_INVALID_ARG, "output width doesnt match to inputB width");
    if (host_pipeline_applies(c, out, x, w, op, cast, M, N, K)) return bgemm_host_pipelined(c, out, x, w, op, cast, M, N, K);
    TRY(stage_in(c, x, &sx, true));
    TRY(stage_in(c, w, &sw, true));
    TRY(stage_in(c, out, &so, !is_dense(out)));
    TRY(bgemm_core(c, &so.t, &sx.t, &sw.t, op, cast, 0));
    TRY(stage_out(c, &so));
    return finish_call(c, any_host);
}

// ------------------------------------------------------------------------------------------ doConvolution
struct ConvShapes {
    uint64_t C, Kout, pixels, taps, rsc;
};

// One spatial dimension of a parity class of dedx: the dX positions cls, cls + stride, ... and the filter taps that
// reach them (the taps t with (cls + pad - t * dil) divisible by the stride; RefIm2Col::internalDoCol2Im,
// mme/mme_reference/im2col.cpp:93-132, visits exactly these).
struct DedxClassDim {
    int count;      // dX positions of the class
    int first_tap, tap_step, taps;
    int lower;      // dY coordinate that the LAST used tap pairs with the class's first position
    int dil;        // dY coordinates between consecutive used taps
};
static DedxClassDim dedx_class_dim(int cls, int stride, int pad, int dil, int taps, int extent) {
    DedxClassDim d;
    memset(&d, 0, sizeof d);
    d.count = extent > cls ? (extent - cls + stride - 1) / stride : 0;
    d.first_tap = -1;
    for (int t = 0; t < taps; ++t)
        if ((((cls + pad - t * dil) % stride) + stride) % stride == 0) { d.first_tap = t; break; }
    int g = dil, h = stride;
    while (h) { const int r = g % h; g = h; h = r; }
    d.tap_step = stride / g;
    d.taps = d.first_tap < 0 ? 0 : (taps - 1 - d.first_tap) / d.tap_step + 1;
    if (d.taps) {
        const int last = d.first_tap + (d.taps - 1) * d.tap_step;
        d.lower = (cls + pad - last * dil) / stride;     // exact
        d.dil = dil * d.tap_step / stride;
    }
    return d;
}

// cls_w / cls_h: dedx of a strided convolution is planned one parity class of dX positions at a time (0, 0 and nothing
// else for stride 1); *cls_empty: no tap reaches the class (its positions stay zero).
static int conv_fast_path(mmeb200_ctx* c, const mmeb200_tensor* x, const mmeb200_tensor* w, const mmeb200_tensor* y,
                          const mmeb200_conv_params* p, int op, GemmJob* job, float* scale, bool* taken, int cls_w = 0, int cls_h = 0,
                          bool* cls_empty = nullptr) {
    *taken = false;
    if (cls_empty) *cls_empty = false;
    const mmeb200_tensor* act = (op == MMEB200_OP_DEDX) ? y : x;   // tensor read through im2col TMA
    const mmeb200_tensor* other = (op == MMEB200_OP_DEDW) ? y : w; // the plain (tiled) operand
    if (p->dim != 2 || x->dims != 4 || y->dims != 4 || w->dims != 4) return 0;
    if (!(act->dtype == DT_BF16 || dtype_is_fp8(act->dtype))) return 0;
    if (dtype_is_fp8(act->dtype) != dtype_is_fp8(other->dtype) || (act->dtype == DT_BF16 && other->dtype != DT_BF16)) return 0;
    const int elem = dtype_size(act->dtype);
    const uint32_t block_k = kRowBytes / elem;
    const uint32_t C = x->sizes[0], Kout = w->sizes[0], S = w->sizes[2], R = w->sizes[3];
    const uint32_t W = x->sizes[1], H = x->sizes[2], B = x->sizes[3];
    const uint32_t Wo = y->sizes[1], Ho = y->sizes[2];
    if (y->sizes[3] != B || w->sizes[1] != C || y->sizes[0] != Kout) return 0;
    if (!is_dense(w) || !is_dense(y) || !is_dense(x)) return 0;
    for (int i = 0; i < 2; ++i)
        if (p->stride[i] < 1 || p->stride[i] > 8 || p->dilation[i] < 1 || p->padding[i] < 0 || p->padding[i] > 127) return 0;
    // output extent must be the one a symmetric padding implies
    auto out_extent = [](int in, int k, int s, int pd, int dl) { return (in + 2 * pd - dl * (k - 1) - 1) / s + 1; };
    if (int(W) + 2 * p->padding[0] - p->dilation[0] * (int(S) - 1) - 1 < 0 || int(H) + 2 * p->padding[1] - p->dilation[1] * (int(R) - 1) - 1 < 0) return 0;
    if (int(Wo) != out_extent(W, S, p->stride[0], p->padding[0], p->dilation[0]) || int(Ho) != out_extent(H, R, p->stride[1], p->padding[1], p->dilation[1])) return 0;
    if ((S - 1) * p->dilation[0] > 255 || (R - 1) * p->dilation[1] > 255) return 0;
    if (span_elems(act) * elem < 131072) return 0;  // small activations take the general path
    if (reinterpret_cast<uintptr_t>(act->data) & 15) return 0;
    // foreign fp8 codes need the decode path
    if (dtype_is_fp8(act->dtype)) {
        const bool act_native = (act->dtype == DT_FP8_143 && act->inf_nan_mode == 2) || (act->dtype == DT_FP8_152 && act->inf_nan_mode == 0);
        const bool oth_native = (other->dtype == DT_FP8_143 && other->inf_nan_mode == 2) || (other->dtype == DT_FP8_152 && other->inf_nan_mode == 0);
        if (!act_native || !oth_native) return 0;
        const int ea = (act->dtype == DT_FP8_143 ? 7 : 15) - int(act->fp_bias);
        const int eb = (other->dtype == DT_FP8_143 ? 7 : 15) - int(other->fp_bias);
        *scale = ldexpf(1.0f, ea + eb);
        job->kind = KIND_F8;
    } else {
        *scale = 1.0f;
        job->kind = KIND_F16;
    }
    const uint32_t fmt_act = act->dtype == DT_BF16 ? 1 : act->dtype == DT_FP8_143 ? 0 : 1;
    const uint32_t fmt_oth = other->dtype == DT_BF16 ? 1 : other->dtype == DT_FP8_143 ? 0 : 1;
    ConvGeom g;
    memset(&g, 0, sizeof g);
    g.dil_w = p->dilation[0]; g.dil_h = p->dilation[1];
    g.taps_w = S; g.taps_h = R;
    int lower[2], upper[2];
    cuuint32_t trav[4] = {1, 1, 1, 1};
    uint32_t chan_box, pix_box;
    if (op == MMEB200_OP_FWD) {
        if (C % block_k) return 0;
        if ((Kout * elem) % 16) return 0;
        g.out_w = Wo; g.out_h = Ho; g.stride_w = p->stride[0]; g.stride_h = p->stride[1];
        g.lower_w = -p->padding[0]; g.lower_h = -p->padding[1];
        lower[0] = g.lower_w; lower[1] = g.lower_h;
        upper[0] = p->padding[0] - (int(S) - 1) * p->dilation[0];
        upper[1] = p->padding[1] - (int(R) - 1) * p->dilation[1];
        trav[1] = p->stride[0]; trav[2] = p->stride[1];
        g.channels = C; g.k_blocks_per_tap = C / block_k;
        chan_box = block_k; pix_box = kBlockM;
        job->M = Wo * Ho * B; job->N = Kout; job->K = S * R * C;
        // B = W as [RSC x Kout], N contiguous
        job->b.ptr = w->data; job->b.elem = elem; job->b.mn_major = true; job->b.inner = Kout; job->b.rows = uint64_t(S) * R * C; job->b.row_stride = Kout;
        job->a.mn_major = false;
    } else if (op == MMEB200_OP_DEDX) {
        if (Kout % block_k) return 0;
        const DedxClassDim dw_ = dedx_class_dim(cls_w, p->stride[0], p->padding[0], p->dilation[0], int(S), int(W));
        const DedxClassDim dh_ = dedx_class_dim(cls_h, p->stride[1], p->padding[1], p->dilation[1], int(R), int(H));
        if (dw_.count == 0 || dh_.count == 0 || dw_.taps == 0 || dh_.taps == 0) {
            if (cls_empty) *cls_empty = true;
            *taken = true;
            return 0;
        }
        g.out_w = dw_.count; g.out_h = dh_.count; g.stride_w = 1; g.stride_h = 1;
        g.lower_w = dw_.lower; g.lower_h = dh_.lower;
        g.dil_w = dw_.dil; g.dil_h = dh_.dil;
        g.taps_w = dw_.taps; g.taps_h = dh_.taps;
        lower[0] = g.lower_w; lower[1] = g.lower_h;
        upper[0] = dw_.count - int(Wo) + g.lower_w;
        upper[1] = dh_.count - int(Ho) + g.lower_h;
        g.flip = 1;
        g.channels = Kout; g.k_blocks_per_tap = Kout / block_k;
        g.b_tap_local = 1;
        g.b_tap_rows = dw_.tap_step * int(C);
        g.b_tap_rows_r = dh_.tap_step * int(S) * int(C);
        g.b_row0 = (dh_.first_tap * int(S) + dw_.first_tap) * int(C);
        if (p->stride[0] != 1 || p->stride[1] != 1) {
            g.out_grid = 1;
            g.out_base = (int64_t(cls_h) * W + cls_w) * C;
            g.out_stride_w = int64_t(p->stride[0]) * C;
            g.out_stride_h = int64_t(p->stride[1]) * W * C;
            g.out_stride_n = int64_t(H) * W * C;
        }
        chan_box = block_k; pix_box = kBlockM;
        job->M = uint32_t(dw_.count) * uint32_t(dh_.count) * B; job->N = C; job->K = uint32_t(dw_.taps * dh_.taps) * Kout;
        // B = W viewed as [RSC rows x Kout], K (=Kout) contiguous: row tap*C + c
        job->b.ptr = w->data; job->b.elem = elem; job->b.mn_major = false; job->b.inner = Kout; job->b.rows = uint64_t(S) * R * C; job->b.row_stride = Kout;
        if ((Kout * elem) % 16) return 0;
        job->a.mn_major = false;
    } else {  // dedw
        const uint32_t group = kRowBytes / elem;
        if (C % group) return 0;
        if ((Kout * elem) % 16) return 0;
        g.out_w = Wo; g.out_h = Ho; g.stride_w = p->stride[0]; g.stride_h = p->stride[1];
        g.lower_w = -p->padding[0]; g.lower_h = -p->padding[1];
        lower[0] = g.lower_w; lower[1] = g.lower_h;
        upper[0] = p->padding[0] - (int(S) - 1) * p->dilation[0];
        upper[1] = p->padding[1] - (int(R) - 1) * p->dilation[1];
        trav[1] = p->stride[0]; trav[2] = p->stride[1];
        g.channels = C; g.pixels_along_k = 1;
        chan_box = group; pix_box = block_k;
        job->M = S * R * C; job->N = Kout; job->K = Wo * Ho * B;
        // B = dY as [pixels x Kout], N contiguous
        job->b.ptr = y->data; job->b.elem = elem; job->b.mn_major = true; job->b.inner = Kout; job->b.rows = uint64_t(Wo) * Ho * B; job->b.row_stride = Kout;
        job->a.mn_major = true;
    }
    for (int i = 0; i < 2; ++i)
        if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return 0;
    if (reinterpret_cast<uintptr_t>(job->b.ptr) & 15) return 0;
    job->a.elem = elem;
    job->a.hw_fmt = fmt_act;
    job->b.hw_fmt = fmt_oth;
    job->conv = g;
    job->a_im2col = true;
    // activation tensor map: (C, W, H, N) of `act`
    TRY(load_driver_entry_points(c));
    cuuint64_t dims[4] = {act->sizes[0], act->sizes[1], act->sizes[2], act->sizes[3]};
    cuuint64_t strides[3] = {uint64_t(act->strides[1]) * elem, uint64_t(act->strides[2]) * elem, uint64_t(act->strides[3]) * elem};
    for (int i = 0; i < 3; ++i)
        if (strides[i] % 16) return 0;
    CUresult r = g_encode_im2col(&job->a_map, tma_dtype(elem), 4, act->data, dims, strides, lower, upper, chan_box, pix_box, trav,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 0;  // geometry outside what the copy engine takes: general path
    *taken = true;
    return 0;
}

int mmeb200_dma(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, int op);

// Convolution tensors with gaps (element strides beyond the dense ones; the reference builds such tensors for its
// strided test cases, mme/mme_verification/common/mme_test_data_gen.cpp:222-298): the operands that are read are
// gathered into dense device copies, the convolution runs on dense tensors, and a strided result is scattered through the
// output's own strides, which leaves the gaps of a caller-owned buffer as they were (dedx writes in place,
// mme_reference_impl.cpp:858-861).
static int conv_with_strided_tensors(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w,
                                     const mmeb200_tensor* y, const mmeb200_conv_params* p, int op, int rounding,
                                     const mmeb200_cast_params* cast) {
    const int base_op = op == MMEB200_OP_TRANSPOSED_DEDX ? MMEB200_OP_DEDX : op == MMEB200_OP_DETERMINISTIC_DEDW ? MMEB200_OP_DEDW : op;
    const mmeb200_tensor* in[3] = {x, w, y};
    const bool read[3] = {base_op != MMEB200_OP_DEDX, base_op != MMEB200_OP_DEDW, base_op != MMEB200_OP_FWD};
    size_t need = 0, off[4] = {0, 0, 0, 0};
    for (int i = 0; i < 3; ++i)
        if (read[i] && !is_dense(in[i])) { off[i] = need; need += (num_elems(in[i]) * dtype_size(in[i]->dtype) + 255) & ~size_t(255); }
    if (!is_dense(out)) { off[3] = need; need += (num_elems(out) * dtype_size(out->dtype) + 255) & ~size_t(255); }
    if (need > c->aux_bytes) {
        CUDA_OK(c, cudaStreamSynchronize(c->stream));
        if (c->aux) CUDA_OK(c, cudaFree(c->aux));
        c->aux = nullptr; c->aux_bytes = 0;
        CUDA_OK(c, cudaMalloc(&c->aux, need));
        c->aux_bytes = need;
    }
    auto dense_view = [&](const mmeb200_tensor* t, size_t offset) {
        mmeb200_tensor d = *t;
        uint32_t acc = 1;
        for (int k = 0; k < 5; ++k) { d.strides[k] = acc; acc *= d.sizes[k]; }
        d.data = static_cast<char*>(c->aux) + offset;
        d.mem_space = MMEB200_MEM_DEVICE;
        return d;
    };
    mmeb200_tensor d[3], d_out;
    for (int i = 0; i < 3; ++i) {
        d[i] = *in[i];
        if (is_dense(in[i])) continue;
        d[i] = dense_view(in[i], read[i] ? off[i] : 0);   // a tensor that is not read only lends its sizes
        if (read[i]) TRY(mmeb200_dma(c, &d[i], in[i], MMEB200_OP_MEMCPY));
    }
    const bool scatter = !is_dense(out);
    if (scatter) d_out = dense_view(out, off[3]);
    TRY(mmeb200_conv(c, scatter ? &d_out : out, &d[0], &d[1], &d[2], p, op, rounding, cast));
    if (scatter) TRY(mmeb200_dma(c, out, &d_out, MMEB200_OP_MEMCPY));
    return 0;
}

int mmeb200_conv(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w, const mmeb200_tensor* y,
                 const mmeb200_conv_params* p, int op, int rounding, const mmeb200_cast_params* cast) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    if (!p) return c->fail(MMEB200_ERR_INVALID_ARG, "null convolution parameters");
    if (out && x && w && y && out->dims >= 1 && out->dims <= 5 && x->dims >= 1 && x->dims <= 5 && w->dims >= 1 && w->dims <= 5 && y->dims >= 1 &&
        y->dims <= 5 && num_elems(out) && num_elems(x) && num_elems(w) && num_elems(y) &&
        (!is_dense(out) || !is_dense(x) || !is_dense(w) || !is_dense(y))) {
        TRY(check_tensor(c, out, "output"));
        TRY(check_tensor(c, x, "x"));
        TRY(check_tensor(c, w, "w"));
        TRY(check_tensor(c, y, "y"));
            return conv_with_strided_tensors(c, out, x, w, y, p, op, rounding, cast);
    }
    if (op == MMEB200_OP_DETERMINISTIC_DEDW) op = MMEB200_OP_DEDW;
    const bool transposed = (op == MMEB200_OP_TRANSPOSED_DEDX);
    if (transposed) op = MMEB200_OP_DEDX;
    if (op != MMEB200_OP_FWD && op != MMEB200_OP_DEDX && op != MMEB200_OP_DEDW) return c->fail(MMEB200_ERR_INVALID_ARG, "invalid operation");
    TRY(check_tensor(c, out, "output"));
    TRY(check_tensor(c, x, "x"));
    TRY(check_tensor(c, w, "w"));
    TRY(check_tensor(c, y, "y"));
    // transposed_dedx hands over the weights with their two fastest dims swapped and S mirrored
    // (mme_reference_impl.cpp:625-647); from here on `w` is the [K, C, S, R, Q] view dedx expects
    const mmeb200_tensor* w_given = w;
    mmeb200_tensor w_view;
    if (transposed) {
        w_view = *w;
        w_view.sizes[0] = w->sizes[1];
        w_view.sizes[1] = w->sizes[0];
        uint32_t acc_stride = 1;
        for (int d = 0; d < 5; ++d) { w_view.strides[d] = acc_stride; acc_stride *= w_view.sizes[d]; }
        w = &w_view;
    }
    if (!cast && out->dtype != DT_FP32 && out->dtype != DT_FP32_IEEE)
        return c->fail(MMEB200_ERR_INVALID_ARG, "without cast parameters the output must be the fp32 accumulator");
    if (p->dim < 1 || p->dim > 3) return c->fail(MMEB200_ERR_INVALID_ARG, "convolution dim %d out of range", p->dim);
    const mmeb200_tensor* shape_of_out = op == MMEB200_OP_FWD ? y : op == MMEB200_OP_DEDX ? x : w;
    for (int d = 0; d < 5; ++d)
        if (out->sizes[d] != shape_of_out->sizes[d]) return c->fail(MMEB200_ERR_INVALID_ARG, "output sizes do not match the operation's result tensor");
    if (w->sizes[1] != x->sizes[0] || y->sizes[0] != w->sizes[0]) return c->fail(MMEB200_ERR_INVALID_ARG, "channel dims of x, w and y disagree");
    arena_reset(c);
    const bool any_host = out->mem_space == MMEB200_MEM_HOST || x->mem_space == MMEB200_MEM_HOST || w_given->mem_space == MMEB200_MEM_HOST ||
                          y->mem_space == MMEB200_MEM_HOST;
    Staged so, sx, sw, sy;
    TRY(stage_in(c, x, &sx, op != MMEB200_OP_DEDX));
    TRY(stage_in(c, w_given, &sw, op != MMEB200_OP_DEDW));
    if (transposed && num_elems(w)) {
        void* flipped = nullptr;
        const int elem = dtype_size(w->dtype);
        TRY(arena_alloc(c, &flipped, num_elems(w) * elem));
        WeightFlipParams fp;
        memset(&fp, 0, sizeof fp);
        fp.n0 = w_given->sizes[0]; fp.n1 = w_given->sizes[1]; fp.S = w_given->sizes[2]; fp.R = w_given->sizes[3]; fp.Q = w_given->sizes[4];
        for (int d = 0; d < 5; ++d) fp.in_stride[d] = w_given->strides[d];
        fp.elem = elem;
        transpose_reverse_s_kernel<<<grid_for(num_elems(w), 256, c->sm_count), 256, 0, c->stream>>>(flipped, sw.t.data, fp);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
        sw.t = w_view;
        sw.t.data = flipped;
        sw.t.mem_space = MMEB200_MEM_DEVICE;
        sw.host = nullptr;
    }
    TRY(stage_in(c, y, &sy, op != MMEB200_OP_FWD));
    TRY(stage_in(c, out, &so, !is_dense(out)));

    CastSpec cs;
    TRY(make_cast_spec(c, out, cast, &cs));
    const bool random = cast && cast_needs_random(cs);
    const bool lfsr_cast = cast && random && cast->rng_kind != MMEB200_RNG_PHILOX && cs.out_dtype != DT_FP32;
    const uint64_t n_out = num_elems(out);
    if (lfsr_cast && !is_dense(out)) return c->fail(MMEB200_ERR_UNSUPPORTED, "LFSR stochastic rounding needs a dense output tensor");

    const uint64_t C = x->sizes[0], Kout = w->sizes[0];
    uint64_t taps = 1, pixels = 1;
    for (int d = 2; d < 5; ++d) taps *= w->sizes[d];
    for (int d = 1; d < 5; ++d) pixels *= y->sizes[d];
    const uint64_t rsc = taps * C;
    if (n_out == 0) return finish_call(c, any_host);
    if (num_elems(x) == 0 || num_elems(w) == 0 || num_elems(y) == 0) {
        CUDA_OK(c, cudaMemsetAsync(so.t.data, 0, so.bytes, c->stream));
        TRY(stage_out(c, &so));
        return finish_call(c, any_host);
    }

    // where the fp32 result of the GEMM goes when the cast cannot be fused
    void* acc = nullptr;
    OutSpec o;
    memset(&o, 0, sizeof o);
    o.bsz[0] = o.bsz[1] = o.bsz[2] = 1;
    auto fused_out = [&](uint64_t ld) {
        o.ptr = so.t.data; o.dtype = cs.out_dtype; o.has_cast = cast != nullptr; o.cast = cs; o.ld = ld;
        o.philox = random && cast->rng_kind == MMEB200_RNG_PHILOX;
        o.seed = cast ? cast->rng_seed : 0; o.offset = cast ? cast->rng_offset : 0;
    };

    // ---- implicit GEMM through im2col-mode TMA (2-D convolutions with friendly geometry)
    GemmJob job;
    float scale = 1.0f;
    bool fast = false;
    const bool dense_out = is_dense(out);
    const bool exact = c->acc_mode == MMEB200_ACC_CHIP_EXACT;
    const bool strided_dedx = op == MMEB200_OP_DEDX && p->dim == 2 && (p->stride[0] != 1 || p->stride[1] != 1);
    if (dense_out && !exact && !(op == MMEB200_OP_DEDX && rounding != RM_NE) && !strided_dedx)
        TRY(conv_fast_path(c, &sx.t, &sw.t, &sy.t, p, op, &job, &scale, &fast));
    if (fast) {
        o.scale = scale;
        const uint64_t ld = (op == MMEB200_OP_DEDX) ? C : Kout;
        if (lfsr_cast) {
            TRY(arena_alloc(c, &acc, n_out * 4));
            o.ptr = acc; o.dtype = DT_FP32; o.has_cast = false; o.ld = ld;
        } else fused_out(ld);
        TRY(run_gemm(c, job, o));
        if (lfsr_cast) TRY(run_cast(c, so.t.data, static_cast<uint32_t*>(acc), n_out, cs, cast));
        TRY(stage_out(c, &so));
        return finish_call(c, any_host);
    }
    // ---- dedx of a strided convolution as implicit GEMMs: the dX positions fall into stride_w x stride_h parity classes,
    //      each reached by its own subset of the taps (im2col.cpp:93-132 adds a tap only where the position divides);
    //      one launch per class reads dY through im2col-mode TMA and stores straight into the class's sub-grid of dX.
    //      No column matrix is materialised.
    if (strided_dedx && dense_out && !exact && rounding == RM_NE && p->stride[0] <= 8 && p->stride[1] <= 8) {
        std::vector<GemmJob> jobs;
        bool all = true, any_empty = false;
        float cls_scale = 1.0f;
        for (int ch = 0; ch < p->stride[1] && all; ++ch)
            for (int cw = 0; cw < p->stride[0] && all; ++cw) {
                GemmJob cj;
                bool taken = false, empty = false;
                TRY(conv_fast_path(c, &sx.t, &sw.t, &sy.t, p, op, &cj, &cls_scale, &taken, cw, ch, &empty));
                all = taken;
                any_empty |= empty;
                if (taken && !empty) jobs.push_back(cj);
            }
        if (all) {
            o.scale = cls_scale;
            if (lfsr_cast) {
                TRY(arena_alloc(c, &acc, n_out * 4));
                o.ptr = acc; o.dtype = DT_FP32; o.has_cast = false; o.ld = C;
            } else fused_out(C);
            // positions that no tap reaches keep the zero the reference fills dX with (im2col.cpp:106)
            if (any_empty) CUDA_OK(c, cudaMemsetAsync(o.ptr, 0, n_out * dtype_size(o.dtype), c->stream));
            for (GemmJob& cj : jobs) TRY(run_gemm(c, cj, o));
            if (lfsr_cast) TRY(run_cast(c, so.t.data, static_cast<uint32_t*>(acc), n_out, cs, cast));
            TRY(stage_out(c, &so));
            return finish_call(c, any_host);
        }
    }
    // ---- general lowering: materialised im2col (fwd, dedw) / col2im (dedx) around the same GEMM
    const mmeb200_tensor* act = (op == MMEB200_OP_DEDX) ? &so.t : &sx.t;  // tensor with the (C,W,H,D,B) geometry
    ConvLowerParams lp;
    memset(&lp, 0, sizeof lp);
    for (int d = 0; d < 5; ++d) {
        lp.act_size[d] = x->sizes[d];
        lp.act_stride[d] = act->strides[d];
        lp.out_size[d] = y->sizes[d];
    }
    for (int i = 0; i < 3; ++i) lp.taps[i] = w->sizes[2 + i];
    for (int i = 0; i < 4; ++i) { lp.stride[i] = p->stride[i]; lp.dil[i] = p->dilation[i]; lp.pad[i] = p->padding[i]; }
    for (int i = p->dim; i < 4; ++i) { lp.stride[i] = 1; lp.dil[i] = 1; lp.pad[i] = 0; }
    for (int i = 0; i < 4; ++i)
        if (lp.stride[i] < 1 || lp.dil[i] < 1) return c->fail(MMEB200_ERR_INVALID_ARG, "convolution stride and dilation must be positive");
    lp.pixels = pixels; lp.rsc = rsc;
    if (!is_dense(w) || !is_dense(y)) return c->fail(MMEB200_ERR_UNSUPPORTED, "strided w / y tensors are not supported in convolutions");

    LogicalOperand la, lb;
    memset(&la, 0, sizeof la);
    memset(&lb, 0, sizeof lb);
    for (int i = 0; i < 3; ++i) { la.bsz[i] = lb.bsz[i] = 1; }
    void* col = nullptr;
    if (op == MMEB200_OP_FWD || op == MMEB200_OP_DEDW) {
        const int elem = dtype_size(x->dtype);
        lp.elem = elem;
        lp.ld = ((rsc * elem + 15) / 16) * 16 / elem;
        TRY(arena_alloc(c, &col, pixels * lp.ld * elem));
        if (lp.ld != rsc) CUDA_OK(c, cudaMemsetAsync(col, 0, pixels * lp.ld * elem, c->stream));
        im2col_kernel<<<grid_for(pixels * rsc, 256, c->sm_count), 256, 0, c->stream>>>(col, sx.t.data, lp);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
    }
    uint64_t M, N;
    if (op == MMEB200_OP_FWD) {
        M = pixels; N = Kout;
        la = {col, x->dtype, int(x->fp_bias), x->inf_nan_mode, pixels, rsc, lp.ld, 1, {1, 1, 1}, {0, 0, 0}};
        lb = {sw.t.data, w->dtype, int(w->fp_bias), w->inf_nan_mode, Kout, rsc, 1, Kout, {1, 1, 1}, {0, 0, 0}};
    } else if (op == MMEB200_OP_DEDW) {
        M = rsc; N = Kout;
        la = {col, x->dtype, int(x->fp_bias), x->inf_nan_mode, rsc, pixels, 1, lp.ld, {1, 1, 1}, {0, 0, 0}};
        lb = {sy.t.data, y->dtype, int(y->fp_bias), y->inf_nan_mode, Kout, pixels, 1, Kout, {1, 1, 1}, {0, 0, 0}};
    } else {
        M = pixels; N = rsc;
        la = {sy.t.data, y->dtype, int(y->fp_bias), y->inf_nan_mode, pixels, Kout, Kout, 1, {1, 1, 1}, {0, 0, 0}};
        lb = {sw.t.data, w->dtype, int(w->fp_bias), w->inf_nan_mode, rsc, Kout, Kout, 1, {1, 1, 1}, {0, 0, 0}};
    }
    mmeb200_tensor ta_whole = (op == MMEB200_OP_DEDX) ? sy.t : sx.t;
    mmeb200_tensor tb_whole = (op == MMEB200_OP_DEDW) ? sy.t : sw.t;
    GemmJob gj, gj_alt;
    float alt_scale = 1.0f;
    bool has_alt = false;
    const uint32_t one3[3] = {1, 1, 1};
    const uint64_t zero3[3] = {0, 0, 0};
    if (!exact) {
        TRY(prepare_pair(c, la, lb, &ta_whole, &tb_whole, &gj, &scale, &gj_alt, &alt_scale, &has_alt));
        gj.M = gj_alt.M = uint32_t(M); gj.N = gj_alt.N = uint32_t(N);
    }
    // both forms of an fp8 GEMM whose operands' convention differs from the tensor cores' are enqueued; the device runs one
    auto run_forms = [&]() -> int {
        o.scale = scale;
        TRY(run_gemm(c, gj, o));
        if (has_alt) {
            o.scale = alt_scale;
            TRY(run_gemm(c, gj_alt, o));
        }
        return 0;
    };
    o.scale = scale;
    if (op == MMEB200_OP_DEDX) {
        // GEMM -> fp32 [pixels x RSC] -> col2im (fp32 dx) -> optional cast
        void* cm = nullptr;
        TRY(arena_alloc(c, &cm, M * N * 4));
        o.ptr = cm; o.dtype = DT_FP32; o.has_cast = false; o.ld = N;
        if (exact) TRY(run_exact_gemm(c, la, lb, M, N, cm, N, one3, zero3));
        else TRY(run_forms());
        lp.ld = N;
        float* dx = nullptr;
        uint64_t dx_span = span_elems(out);
        if (!cast) dx = static_cast<float*>(so.t.data);
        else {
            TRY(arena_alloc(c, reinterpret_cast<void**>(&dx), dx_span * 4));
        }
        if (!dense_out && cast) return c->fail(MMEB200_ERR_UNSUPPORTED, "fused cast needs a dense dedx output");
        col2im_kernel<<<grid_for(n_out, 256, c->sm_count), 256, 0, c->stream>>>(dx, static_cast<const float*>(cm), lp, rounding);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
        if (cast) TRY(run_cast(c, so.t.data, reinterpret_cast<uint32_t*>(dx), n_out, cs, cast));
    } else {
        // rows of the GEMM result are rows of the (dense or row-strided) output tensor
        if (!dense_out) {
            // only a row pitch (strides[1]) is honoured here
            uint64_t accs = out->strides[1] * out->sizes[1];
            for (int d = 2; d < 5; ++d) {
                if (out->sizes[d] != 1 && out->strides[d] != accs) return c->fail(MMEB200_ERR_UNSUPPORTED, "output strides beyond the row pitch are not supported");
                accs *= out->sizes[d];
            }
        }
        const uint64_t ld = out->strides[1];
        if (exact && c->pending_peer) {
            // bit-exact partial dW into scratch, then the same exchange as the tensor-core path
            const mmeb200_peer_group* peer = c->pending_peer;
            c->pending_peer = nullptr;
            if (cast || !dense_out) return c->fail(MMEB200_ERR_UNSUPPORTED, "the fused dedw exchange needs a dense fp32 result");
            void* part = nullptr;
            TRY(arena_alloc(c, &part, M * N * 4));
            TRY(run_exact_gemm(c, la, lb, M, N, part, N, one3, zero3));
            TRY(run_peer_exchange(c, peer, static_cast<const float*>(part), 1, M * N, 1.0f, static_cast<float*>(so.t.data)));
        } else if (exact) {
            if (!cast) TRY(run_exact_gemm(c, la, lb, M, N, so.t.data, ld, one3, zero3));
            else {
                if (!dense_out) return c->fail(MMEB200_ERR_UNSUPPORTED, "a cast after bit-exact accumulation needs a dense output tensor");
                TRY(arena_alloc(c, &acc, n_out * 4));
                TRY(run_exact_gemm(c, la, lb, M, N, acc, N, one3, zero3));
                TRY(run_cast(c, so.t.data, static_cast<uint32_t*>(acc), n_out, cs, cast));
            }
        } else if (lfsr_cast) {
            TRY(arena_alloc(c, &acc, n_out * 4));
            o.ptr = acc; o.dtype = DT_FP32; o.has_cast = false; o.ld = N;
            TRY(run_forms());
            TRY(run_cast(c, so.t.data, static_cast<uint32_t*>(acc), n_out, cs, cast));
        } else {
            fused_out(ld);
            TRY(run_forms());
        }
    }
    TRY(stage_out(c, &so));
    return finish_call(c, any_host);
}

// ------------------------------------------------------------------------------------------ TensorComparator
int mmeb200_compare(mmeb200_ctx* c, const mmeb200_tensor* a, const mmeb200_tensor* b, unsigned cd_size, unsigned num_partials,
                    int bit_exact, mmeb200_compare_result* result) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    if (!result) return c->fail(MMEB200_ERR_INVALID_ARG, "null result");
    TRY(check_tensor(c, a, "a"));
    TRY(check_tensor(c, b, "b"));
    if (a->dtype != b->dtype) return c->fail(MMEB200_ERR_INVALID_ARG, "Element type of sim tensors should match to perform proper comparison");
    if (num_partials < 1 || num_elems(a) != num_elems(b) * num_partials) return c->fail(MMEB200_ERR_INVALID_ARG, "tensor sizes do not match");
    if (!is_dense(a) || !is_dense(b)) return c->fail(MMEB200_ERR_UNSUPPORTED, "the comparator takes dense tensors");
    if (num_partials > 1 && !(b->dtype == DT_FP32 || b->dtype == DT_FP32_IEEE || b->dtype == DT_BF16))
        return c->fail(MMEB200_ERR_UNSUPPORTED, "partial sums are compared for fp32 and bf16 tensors only");
    arena_reset(c);
    Staged sa, sb;
    TRY(stage_in(c, a, &sa, true));
    TRY(stage_in(c, b, &sb, true));
    unsigned long long* d = nullptr;
    TRY(arena_alloc(c, reinterpret_cast<void**>(&d), 16));
    const unsigned long long init[2] = {0ull, ~0ull};
    CUDA_OK(c, cudaMemcpyAsync(d, init, 16, cudaMemcpyHostToDevice, c->stream));
    CompareParams p;
    memset(&p, 0, sizeof p);
    p.a = sa.t.data; p.b = sb.t.data; p.n = num_elems(b); p.num_partials = num_partials; p.elem = dtype_size(b->dtype);
    p.bit_exact = bit_exact;
    const int dt = (b->dtype == DT_FP32_IEEE || b->dtype == DT_TF32) ? DT_FP32 : b->dtype;
    p.spec = make_compare_spec(dt, int(b->fp_bias), b->inf_nan_mode, cd_size);
    p.mismatches = d;
    if (p.n) {
        compare_kernel<<<grid_for((p.n + 3) / 4, 256, c->sm_count), 256, 0, c->stream>>>(p);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
    }
    unsigned long long host[2];
    CUDA_OK(c, cudaMemcpyAsync(host, d, 16, cudaMemcpyDeviceToHost, c->stream));
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    result->mismatches = host[0];
    result->first_index = host[1];
    return collect_status(c);
}

// ------------------------------------------------------------------------------------------ tensor generator
// Largest finite value of a tensor's type: what the type's constructor makes of FLT_MAX with clipping on
// (fp8.h:107-129 max(); bf16 / fp32: the largest normal).
static float type_max_value(const mmeb200_tensor* t) {
    uint32_t bits;
    switch (t->dtype) {
        case DT_FP8_143:
        case DT_FP8_152: {
            const int ew = t->dtype == DT_FP8_143 ? 4 : 5;
            const uint32_t code = f32_to_fp8(0x7F7FFFFFu, ew, int(t->fp_bias), RM_NE, 0u, false, true, false, false, t->inf_nan_mode);
            bits = fp8_decode(code, ew, int(t->fp_bias), t->inf_nan_mode);
            break;
        }
        case DT_BF16: bits = 0x7F7F0000u; break;
        case DT_TF32: bits = 0x7F7FE000u; break;
        default: bits = 0x7F7FFFFFu; break;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

int mmeb200_generate(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_generate_params* gp) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    if (!gp) return c->fail(MMEB200_ERR_INVALID_ARG, "null generator parameters");
    TRY(check_tensor(c, out, "output"));
    if (!is_dense(out)) return c->fail(MMEB200_ERR_UNSUPPORTED, "the generator fills dense tensors");
    if (gp->kind < MMEB200_GEN_UNIFORM || gp->kind > MMEB200_GEN_REDUCTION_PACKING) return c->fail(MMEB200_ERR_INVALID_ARG, "generator kind %d is not valid", gp->kind);
    if (gp->min_value > gp->max_value) return c->fail(MMEB200_ERR_INVALID_ARG, "min value is larger then max value");
    if (gp->kind == MMEB200_GEN_REDUCTION_PACKING && (gp->packing == 0 || gp->level == 0)) return c->fail(MMEB200_ERR_INVALID_ARG, "packing and level must be positive");
    arena_reset(c);
    Staged so;
    TRY(stage_in(c, out, &so, false));
    GenerateParams g;
    memset(&g, 0, sizeof g);
    const float tmax = type_max_value(out);
    g.out = so.t.data; g.n = num_elems(out); g.kind = gp->kind;
    g.lo = std::max(gp->min_value, -tmax); g.hi = std::min(gp->max_value, tmax);
    if (gp->kind == MMEB200_GEN_UNIT) { g.lo = gp->min_value; g.hi = gp->max_value; }   // the reference passes these two through unclamped
    g.mean = gp->mean; g.std_dev = gp->std_dev; g.seed = gp->seed;
    g.packing = gp->packing; g.row_size = gp->packing * gp->level;
    g.out_dtype = out->dtype == DT_FP32_IEEE ? DT_FP32 : out->dtype;
    if (g.out_dtype != DT_FP32 && g.out_dtype != DT_TF32) TRY(make_cast_spec(c, out, nullptr, &g.cast));
    if (g.n) {
        generate_kernel<<<grid_for((g.n + 3) / 4, 256, c->sm_count), 256, 0, c->stream>>>(g);
        c->launches++;
        CUDA_OK(c, cudaGetLastError());
    }
    TRY(stage_out(c, &so));
    return finish_call(c, out->mem_space == MMEB200_MEM_HOST);
}

// ------------------------------------------------------------------------------------------ dedw + exchange
size_t mmeb200_peer_exchange_bytes(uint64_t n_floats, int world) {
    if (world < 1 || world > MMEB200_MAX_PEERS) return 0;
    return size_t(2) * size_t(world) * peer_segment_floats(n_floats, world) * sizeof(float);
}
int mmeb200_peer_alloc(mmeb200_ctx* c, size_t bytes, void** dev_ptr, unsigned char handle[MMEB200_PEER_HANDLE_BYTES]) {
    if (!c || !dev_ptr || !handle || bytes == 0) return MMEB200_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == MMEB200_PEER_HANDLE_BYTES, "handle size");
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaMalloc(dev_ptr, bytes));
    CUDA_OK(c, cudaMemset(*dev_ptr, 0, bytes));
    cudaIpcMemHandle_t h;
    CUDA_OK(c, cudaIpcGetMemHandle(&h, *dev_ptr));
    memcpy(handle, &h, sizeof h);
    return 0;
}
int mmeb200_peer_open(mmeb200_ctx* c, const unsigned char handle[MMEB200_PEER_HANDLE_BYTES], void** dev_ptr) {
    if (!c || !dev_ptr || !handle) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    CUDA_OK(c, cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}
int mmeb200_peer_close(mmeb200_ctx* c, void* dev_ptr) {
    if (!c || !dev_ptr) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    CUDA_OK(c, cudaStreamSynchronize(c->stream));
    CUDA_OK(c, cudaIpcCloseMemHandle(dev_ptr));
    return 0;
}
int mmeb200_conv_dedw_allreduce(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w,
                                const mmeb200_tensor* y, const mmeb200_conv_params* params, const mmeb200_peer_group* g) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    if (!g || !out) return c->fail(MMEB200_ERR_INVALID_ARG, "null peer group or output");
    if (g->world < 1 || g->world > MMEB200_MAX_PEERS || g->rank < 0 || g->rank >= g->world)
        return c->fail(MMEB200_ERR_INVALID_ARG, "peer group: rank %d of %d is not valid", g->rank, g->world);
    for (int i = 0; i < g->world; ++i)
        if (!g->slots[i] || !g->flags[i]) return c->fail(MMEB200_ERR_INVALID_ARG, "peer group: rank %d has no slot buffer or flag", i);
    if (out->dtype != DT_FP32 || !is_dense(out)) return c->fail(MMEB200_ERR_INVALID_ARG, "the summed dW must be a dense fp32 tensor");
    mmeb200_peer_group group = *g;
    if (out->mem_space != MMEB200_MEM_DEVICE) group.deferred_output = 0;   // a host output is copied back before the call returns
    c->pending_peer = &group;
    const int rc = mmeb200_conv(c, out, x, w, y, params, MMEB200_OP_DEDW, RM_NE, nullptr);
    const bool consumed = c->pending_peer == nullptr;
    c->pending_peer = nullptr;
    if (rc == 0 && !consumed)   // a path that produced only this rank's partial: the peers would wait for nothing
        return c->fail(MMEB200_ERR_UNSUPPORTED, "this dedw took a path without the cross-GPU exchange (empty tensors?)");
    return rc;
}

// ------------------------------------------------------------------------------------------ doActivation
int mmeb200_activation(mmeb200_ctx* c, mmeb200_tensor* out, mmeb200_tensor* acc, const mmeb200_cast_params* cast) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    TRY(check_tensor(c, out, "output"));
    TRY(check_tensor(c, acc, "acc"));
    if (!cast) return c->fail(MMEB200_ERR_INVALID_ARG, "null cast parameters");
    if (acc->dtype != DT_FP32) return c->fail(MMEB200_ERR_INVALID_ARG, "acc element type should be fp32");
    if (acc->dims != out->dims) return c->fail(MMEB200_ERR_INVALID_ARG, "dims number of outputTensor doesnt match acc output");
    for (int d = 0; d < 5; ++d)
        if (acc->sizes[d] != out->sizes[d]) return c->fail(MMEB200_ERR_INVALID_ARG, "sizes of output Tensot doesnt match acc output");
    if (!is_dense(acc) || !is_dense(out)) return c->fail(MMEB200_ERR_INVALID_ARG, "input and output should be flattened");
    arena_reset(c);
    const bool any_host = out->mem_space == MMEB200_MEM_HOST || acc->mem_space == MMEB200_MEM_HOST;
    Staged so, sa;
    TRY(stage_in(c, acc, &sa, true));
    TRY(stage_in(c, out, &so, false));
    CastSpec cs;
    TRY(make_cast_spec(c, out, cast, &cs));
    TRY(run_cast(c, so.t.data, static_cast<uint32_t*>(sa.t.data), num_elems(acc), cs, cast));
    if (cs.relu) TRY(stage_out(c, &sa));  // the reference applies ReLU to the accumulator in place
    TRY(stage_out(c, &so));
    return finish_call(c, any_host);
}

// ------------------------------------------------------------------------------------------ doMemoryWrite
int mmeb200_memory_write(mmeb200_ctx* c, mmeb200_tensor* mem, const mmeb200_tensor* mme_out, int red_op, int red_rm, int clip_fp) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    TRY(check_tensor(c, mem, "memory"));
    TRY(check_tensor(c, mme_out, "mmeOut"));
    if (num_elems(mem) != num_elems(mme_out) || mem->dtype != mme_out->dtype) return c->fail(MMEB200_ERR_INVALID_ARG, "memory and mmeOut differ in size or type");
    if (!is_dense(mem) || !is_dense(mme_out)) return c->fail(MMEB200_ERR_UNSUPPORTED, "memory write needs dense tensors");
    arena_reset(c);
    const bool any_host = mem->mem_space == MMEB200_MEM_HOST || mme_out->mem_space == MMEB200_MEM_HOST;
    Staged sm, so;
    const uint64_t n = num_elems(mem);
    if (red_op == MMEB200_RED_NONE) {
        TRY(stage_in(c, mme_out, &so, true));
        TRY(stage_in(c, mem, &sm, false));
        CUDA_OK(c, cudaMemcpyAsync(sm.t.data, so.t.data, n * dtype_size(mem->dtype), cudaMemcpyDeviceToDevice, c->stream));
    } else if (red_op >= MMEB200_RED_ADD && red_op <= MMEB200_RED_MAX_0 && (mem->dtype == DT_FP32 || mem->dtype == DT_BF16 || mem->dtype == DT_FP8_152)) {
        if (red_rm < 0 || red_rm > 3) return c->fail(MMEB200_ERR_INVALID_ARG, "reduction rounding mode %d is not valid", red_rm);
        TRY(stage_in(c, mme_out, &so, true));
        TRY(stage_in(c, mem, &sm, true));
        if (n && mem->dtype == DT_FP32) {
            memory_write_f32_kernel<<<grid_for((n + 7) / 8, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<uint32_t*>(sm.t.data),
                                                                                         static_cast<const uint32_t*>(so.t.data), n,
                                                                                         red_op, red_rm, clip_fp);
            c->launches++;
        } else if (n && mem->dtype == DT_FP8_152) {
            // the reference's fp8 RMW type is 1-5-2 with the hardware bias and the full Inf/NaN convention (fs_fma.cpp:2410-2435)
            if (mem->fp_bias != 15 || mme_out->fp_bias != 15 || mem->inf_nan_mode != 0)
                return c->fail(MMEB200_ERR_UNSUPPORTED, "fp8_152 reductions are defined for exponent bias 15 and the full Inf/NaN convention");
            memory_write_fp8_152_kernel<<<grid_for((n + 15) / 16, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<uint8_t*>(sm.t.data),
                                                                                               static_cast<const uint8_t*>(so.t.data), n,
                                                                                               red_op, red_rm, clip_fp);
            c->launches++;
        } else if (n) {
            memory_write_bf16_kernel<<<grid_for((n + 7) / 8, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<uint16_t*>(sm.t.data),
                                                                                          static_cast<const uint16_t*>(so.t.data), n,
                                                                                          red_op, red_rm, clip_fp);
            c->launches++;
        }
    } else {
        return c->fail(MMEB200_ERR_UNSUPPORTED, "reduction op %d on data type %d is not implemented", red_op, mem->dtype);
    }
    TRY(stage_out(c, &sm));
    return finish_call(c, any_host);
}

// ------------------------------------------------------------------------------------------ conversions
int mmeb200_convert(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* in, const mmeb200_cast_params* cast) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    TRY(check_tensor(c, out, "output"));
    TRY(check_tensor(c, in, "input"));
    if (num_elems(out) != num_elems(in)) return c->fail(MMEB200_ERR_INVALID_ARG, "element counts differ");
    if (!is_dense(out) || !is_dense(in)) return c->fail(MMEB200_ERR_UNSUPPORTED, "conversions need dense tensors");
    arena_reset(c);
    const bool any_host = out->mem_space == MMEB200_MEM_HOST || in->mem_space == MMEB200_MEM_HOST;
    const uint64_t n = num_elems(in);
    Staged so, si;
    TRY(stage_in(c, in, &si, true));
    TRY(stage_in(c, out, &so, false));
    const bool in_f32 = in->dtype == DT_FP32 || in->dtype == DT_FP32_IEEE;
    const bool out_f32 = out->dtype == DT_FP32 || out->dtype == DT_FP32_IEEE;
    if (!in_f32 && out_f32) {
        if (n) {
            decode_kernel<<<grid_for(n, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<uint32_t*>(so.t.data), si.t.data, n, in->dtype,
                                                                               int(in->fp_bias), in->inf_nan_mode);
            c->launches++;
        }
    } else if (in_f32) {
        CastSpec cs;
        mmeb200_cast_params dflt;
        memset(&dflt, 0, sizeof dflt);
        const mmeb200_cast_params* cp = cast ? cast : &dflt;
        TRY(make_cast_spec(c, out, cp, &cs));
        cs.relu = 0;
        // the input must stay untouched: ReLU is off, so run_cast only reads it
        TRY(run_cast(c, so.t.data, static_cast<uint32_t*>(si.t.data), n, cs, cp));
    } else {
        return c->fail(MMEB200_ERR_UNSUPPORTED, "conversion from data type %d to %d goes through fp32", in->dtype, out->dtype);
    }
    TRY(stage_out(c, &so));
    return finish_call(c, any_host);
}

// ------------------------------------------------------------------------------------------ doDma
int mmeb200_dma(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, int op) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    TRY(check_tensor(c, out, "output"));
    TRY(check_tensor(c, x, "x"));
    if (op == MMEB200_OP_GEMM_TRANSPOSE) op = MMEB200_OP_TRANS;   // same transposition in the calculator
    if (op != MMEB200_OP_MEMCPY && op != MMEB200_OP_TRANS) return c->fail(MMEB200_ERR_INVALID_ARG, "invalid operation");
    if (dtype_size(out->dtype) != dtype_size(x->dtype)) return c->fail(MMEB200_ERR_INVALID_ARG, "element sizes differ");
    const bool tr = op == MMEB200_OP_TRANS;
    for (int d = 0; d < 5; ++d) {
        const int od = tr ? (d == 0 ? 1 : d == 1 ? 0 : d) : d;
        if (out->sizes[od] != x->sizes[d]) return c->fail(MMEB200_ERR_INVALID_ARG, "output sizes do not match the input");
    }
    arena_reset(c);
    const bool any_host = out->mem_space == MMEB200_MEM_HOST || x->mem_space == MMEB200_MEM_HOST;
    Staged so, sx;
    TRY(stage_in(c, x, &sx, true));
    TRY(stage_in(c, out, &so, !is_dense(out)));
    CopyParams cp;
    memset(&cp, 0, sizeof cp);
    cp.elem = dtype_size(x->dtype);
    for (int d = 0; d < 5; ++d) {
        const int od = tr ? (d == 0 ? 1 : d == 1 ? 0 : d) : d;
        cp.size[d] = x->sizes[d];
        cp.in_stride[d] = x->strides[d];
        cp.out_stride[d] = out->strides[od];
    }
    const uint64_t n = num_elems(x);
    if (n) {
        strided_copy_kernel<<<grid_for(n, 256, c->sm_count), 256, 0, c->stream>>>(so.t.data, sx.t.data, cp);
        c->launches++;
    }
    TRY(stage_out(c, &so));
    return finish_call(c, any_host);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------ split-K GEMM without allocations
// The split-K path above keeps its fp32 partial sums in scratch memory that the context obtains
// with cudaMalloc on demand. Some callers may not allocate at the moment they need a GEMM: code
// that runs under a framework's memory pool and has been handed exactly its inputs and outputs, a
// latency-critical loop that must not hit the allocator's lock, or a process whose memory budget
// was fixed at start-up. For them the same kernels run with the partial sums in the fixed array
// below, which is part of the library image: every GPU that loads the library holds these 16 MiB
// until the process exits.
constexpr size_t kStaticSplitKBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_static_splitk_ws[kStaticSplitKBytes];
// Device address of g_static_splitk_ws per CUDA ordinal. In host code the array's name is only a
// handle for the runtime, never an address a kernel may use; cudaGetSymbolAddress translates it.
static void* g_static_splitk_addr[64] = {};

extern "C" int mmeb200_gemm_splitk_static(mmeb200_ctx* c, mmeb200_tensor* out, const mmeb200_tensor* x, const mmeb200_tensor* w,
                                          int op, int splits) {
    if (!c) return MMEB200_ERR_INVALID_ARG;
    cudaSetDevice(c->device);
    TRY(check_tensor(c, out, "output"));
    TRY(check_tensor(c, x, "x"));
    TRY(check_tensor(c, w, "w"));
    if (op < MMEB200_OP_AB || op > MMEB200_OP_ATBT) return c->fail(MMEB200_ERR_INVALID_ARG, "operation %d is not a gemm operation", op);
    if (out->mem_space != MMEB200_MEM_DEVICE || x->mem_space != MMEB200_MEM_DEVICE || w->mem_space != MMEB200_MEM_DEVICE)
        return c->fail(MMEB200_ERR_INVALID_ARG, "the allocation-free gemm takes device-resident tensors only (staging host tensors would allocate)");
    if (out->dtype != DT_FP32) return c->fail(MMEB200_ERR_INVALID_ARG, "the allocation-free gemm writes the fp32 accumulator");
    for (int d = 2; d < 5; ++d)
        if (out->sizes[d] != 1 || x->sizes[d] != 1 || w->sizes[d] != 1) return c->fail(MMEB200_ERR_UNSUPPORTED, "the allocation-free gemm is 2-D (no batch dims)");
    const bool x8 = dtype_is_fp8(x->dtype), w8 = dtype_is_fp8(w->dtype);
    auto native8 = [](const mmeb200_tensor* t) { return (t->dtype == DT_FP8_143 && t->inf_nan_mode == 2) || (t->dtype == DT_FP8_152 && t->inf_nan_mode == 0); };
    if (!((x->dtype == DT_BF16 && w->dtype == DT_BF16) || (x8 && w8 && native8(x) && native8(w))))
        return c->fail(MMEB200_ERR_UNSUPPORTED, "the allocation-free gemm takes bf16 x bf16, or fp8 operands whose Inf/NaN convention the tensor cores share "
                                                "(1-4-3 'minimal', 1-5-2 'full'); other formats need converted copies, i.e. scratch allocations");
    const bool tA = (op == MMEB200_OP_ATB || op == MMEB200_OP_ATBT), tB = (op == MMEB200_OP_ABT || op == MMEB200_OP_ATBT);
    const uint64_t M = tA ? x->sizes[0] : x->sizes[1], K = tA ? x->sizes[1] : x->sizes[0];
    const uint64_t Kb = tB ? w->sizes[0] : w->sizes[1], N = tB ? w->sizes[1] : w->sizes[0];
    if (M == 0 || N == 0 || K == 0) return c->fail(MMEB200_ERR_INVALID_ARG, "empty operands");
    if (K != Kb) return c->fail(MMEB200_ERR_INVALID_ARG, "Common dim doesnt match between input A\\B");
    if (out->sizes[0] != N || out->sizes[1] != M) return c->fail(MMEB200_ERR_INVALID_ARG, "output width doesnt match to inputB width");
    const int elem = dtype_size(x->dtype);
    const uint32_t block_k = kRowBytes / elem;
    const uint32_t num_k_blocks = uint32_t((K + block_k - 1) / block_k);
    if (splits < 2 || splits > 64 || uint32_t(splits) > num_k_blocks)
        return c->fail(MMEB200_ERR_INVALID_ARG, "splits must be in [2, min(64, %u k-blocks)], got %d", num_k_blocks, splits);
    if (((num_k_blocks + splits - 1) / splits) * uint32_t(splits - 1) >= num_k_blocks)
        return c->fail(MMEB200_ERR_INVALID_ARG, "%d splits of %u k-blocks would leave a split empty", splits, num_k_blocks);
    const uint64_t need = uint64_t(splits) * M * N * 4;
    if (need > kStaticSplitKBytes)
        return c->fail(MMEB200_ERR_INVALID_ARG, "splits * M * N * 4 = %llu bytes exceeds the fixed %llu-byte workspace of the allocation-free gemm",
                       (unsigned long long) need, (unsigned long long) kStaticSplitKBytes);

    // one-time set-up per device: translate the symbol to its device address (this device is current)
    if (c->device < 0 || c->device >= 64) return c->fail(MMEB200_ERR_INVALID_ARG, "device ordinal %d out of range", c->device);
    if (!g_static_splitk_addr[c->device]) {
        void* addr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&addr, g_static_splitk_ws);
        if (e != cudaSuccess || !addr) return c->fail(MMEB200_ERR_CUDA, "cudaGetSymbolAddress(static split-K workspace): %s", cudaGetErrorString(e));
        g_static_splitk_addr[c->device] = addr;
    }
    void* ws = g_static_splitk_addr[c->device];

    LogicalOperand la, lb;
    la.ptr = x->data; la.dtype = x->dtype; la.bias = int(x->fp_bias); la.mode = x->inf_nan_mode;
    la.mn = M; la.k = K; la.mn_stride = tA ? 1 : x->strides[1]; la.k_stride = tA ? x->strides[1] : 1;
    lb.ptr = w->data; lb.dtype = w->dtype; lb.bias = int(w->fp_bias); lb.mode = w->inf_nan_mode;
    lb.mn = N; lb.k = K; lb.mn_stride = tB ? w->strides[1] : 1; lb.k_stride = tB ? 1 : w->strides[1];
    for (int i = 0; i < 3; ++i) { la.bsz[i] = lb.bsz[i] = 1; la.bstride[i] = lb.bstride[i] = 0; }
    TmaOperand a, b;
    if (native_operand(la, &a) != 0 || !tma_compatible(a) || native_operand(lb, &b) != 0 || !tma_compatible(b))
        return c->fail(MMEB200_ERR_UNSUPPORTED, "operands must be 16-byte aligned with row pitches that are multiples of 16 bytes "
                                                "(anything else needs a repacked copy, i.e. a scratch allocation)");
    float scale = 1.0f;
    uint32_t kind = KIND_F16;
    if (x8) {
        kind = KIND_F8;
        a.hw_fmt = x->dtype == DT_FP8_143 ? 0 : 1;
        b.hw_fmt = w->dtype == DT_FP8_143 ? 0 : 1;
        scale = ldexpf(1.0f, ((x->dtype == DT_FP8_143 ? 7 : 15) - int(x->fp_bias)) + ((w->dtype == DT_FP8_143 ? 7 : 15) - int(w->fp_bias)));
    } else {
        a.hw_fmt = b.hw_fmt = 1;
    }

    GemmParams p;
    memset(&p, 0, sizeof p);
    p.M = uint32_t(M); p.N = uint32_t(N); p.K = uint32_t(K);
    p.elem_bytes = elem; p.block_k = block_k; p.num_k_blocks = num_k_blocks;
    p.m_tiles = uint32_t((M + kBlockM - 1) / kBlockM);
    p.batches = 1;
    for (int i = 0; i < 3; ++i) { p.bsz[i] = 1; p.a_bcast[i] = 1; p.b_bcast[i] = 1; }
    p.a_mn_major = a.mn_major; p.b_mn_major = b.mn_major; p.a_mode = A_TILED;
    constexpr int block_n = 128;
    p.n_tiles = uint32_t((N + block_n - 1) / block_n);
    p.split_k = uint32_t(splits);
    p.raster_gm = 16;
    p.idesc = make_instr_desc(a.hw_fmt, b.hw_fmt, a.mn_major, b.mn_major, kBlockM, block_n);
    p.status = c->d_status;
    p.scale = 1.0f; p.out_dtype = DT_FP32; p.has_cast = 0; p.epi_mode = EPI_F32;
    p.out = ws;   // every (split, tile) overwrites its whole region of the workspace: nothing has to start at zero
    TRY(encode_tiled(c, &p.tm_a, a, a.mn_major ? kRowBytes / elem : block_k, a.mn_major ? block_k : kBlockM));
    TRY(encode_tiled(c, &p.tm_b, b, b.mn_major ? kRowBytes / elem : block_k, b.mn_major ? block_k : block_n));
    const uint64_t tiles = uint64_t(p.m_tiles) * p.n_tiles * splits;
    const unsigned grid = unsigned(std::min<uint64_t>(tiles, uint64_t(c->sm_count)));
    TRY(launch_status(c, launch_gemm_single(launch_env(c), kind, 128, p, grid)));
    ReduceOut r;
    memset(&r, 0, sizeof r);
    r.out = out->data; r.out_dtype = DT_FP32; r.has_cast = 0; r.out_ld = out->strides[1];
    for (int i = 0; i < 3; ++i) r.bsz[i] = 1;
    r.M = p.M; r.N = p.N; r.batches = 1; r.splits = uint32_t(splits); r.scale = scale;
    splitk_reduce_kernel<<<grid_for(M * N, 256, c->sm_count), 256, 0, c->stream>>>(static_cast<const float*>(ws), r);
    c->launches++;
    CUDA_OK(c, cudaGetLastError());
    return 0;
}
