// CTA-pair variant of the tcgen05 GEMM (tiled and im2col operands, optional split-K): two CTAs of one cluster
// compute one 256 x 256 output tile with a single tcgen05.mma.cta_group::2 per 32 bytes of K. Each CTA
// stages its own 128 rows of A and only its half of B (128 of the tile's 256 columns), so a stage is
// 32 KB instead of 48 KB: B's shared-memory traffic halves and the ring gets 6 stages.
//
// Roles per CTA are the same as in gemm_tcgen05_kernel, with these differences:
//   * full[stage] lives in the even-ranked ("leader") CTA. Its two arrivals are the leader's A and B
//     producer, each announcing the bytes of BOTH CTAs' loads of that operand; the partner's
//     producers only issue their loads, which complete on the leader's barrier
//     (the cta_group::2 form of the tiled load; each CTA fetches its own tile). The partner never makes a remote
//     arrival per stage: a release-ordered remote arrival costs a round trip between the SMs.
//   * only the leader's MMA thread issues; its commits arrive on empty[stage] / tmem_full[acc] of
//     BOTH CTAs (tcgen05.commit ... multicast::cluster).
//   * tmem_empty[acc] lives in the leader and counts one arrival per epilogue warp of both CTAs.
//   * tensor memory is allocated and freed by one warp of each CTA with the cta_group::2 forms; the
//     cluster synchronises after set-up and before tear-down.
// Every wait is bounded as in the single-CTA kernel; after a wait gives up each role leaves its loop,
// and all threads still meet at the final cluster barrier.
#pragma once
#include "gemm_sm100.cuh"

namespace mmeb200 {

constexpr uint64_t kSkWaitLimitNs = 500000000ull;   // a cut tile's other pieces are a few pieces' time away at most
constexpr int kPairBlockN = 256;       // most columns a pair's tile can have (p.tile_n of them are used); each CTA stages half

// EPI_GROUPS = 1: four epilogue warps drain the CTA's 128 x 256 accumulator (six operand stages).
// EPI_GROUPS = 2: eight epilogue warps, each group of four takes half of the columns (five stages; the
// second group's output staging buffers take the place of the sixth). For tiles with so few k blocks
// that the epilogue, not the MMA, sets the pace.
template <int EPI_GROUPS>
struct PairSmem {
    static constexpr int kStages = EPI_GROUPS == 1 ? 6 : 5;
    static constexpr int kABytes = kBlockM * kRowBytes;
    static constexpr int kBBytes = (kPairBlockN / 2) * kRowBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kOutStageBytes = EPI_GROUPS * 2 * kBlockM * kRowBytes;
    static constexpr int kTotal = kStages * kStageBytes + kOutStageBytes + kBarrierBytes;   // see GemmSmem::kTotal
    static constexpr int kThreads = 128 + 128 * EPI_GROUPS;
};

// p.m_tiles counts 256-row tiles here; p.n_tiles counts tiles of p.tile_n columns. The planner narrows tile_n (a
// multiple of 32) when that fills the last wave of tiles better: one MMA then covers 256 x tile_n, CTA `rank` stages the
// columns from rank * tile_n / 2 on (whole 128-byte groups of an MN-major B: up to 16 bytes' worth of columns more than it
// needs), and the epilogue leaves the columns after tile_n to the next tile.
// CUT: the instantiation that can run a cut tail (p.sk_tiles != 0); the others carry none of its code.
template <int KIND, int EPI_GROUPS, bool CUT = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairSmem<EPI_GROUPS>::kThreads, 1)
    gemm_tcgen05_pair_kernel(const __grid_constant__ GemmParams p) {
    using S = PairSmem<EPI_GROUPS>;
    constexpr int STAGES = S::kStages;
    if (p.pred) griddep_wait();   // the predicate word comes from an earlier kernel of the stream
    if (launch_is_predicated_off(p.pred, p.pred_nonzero)) return;   // uniform over the grid (both CTAs of every pair)
    griddep_launch_dependents();   // all CTAs of this grid are resident: what frees up may go to the next kernel
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (smem_u32(smem) & 1023u) {   // uniform over the cluster: both CTAs see the same offset
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, SMEM_MISALIGNED);
        return;
    }
    if (p.sk_tiles && (!CUT || (gridDim.x >> 1) <= p.sk_tiles)) {   // nobody would compute the cut tiles' pieces
        if (threadIdx.x == 0) atomicCAS(p.status, 0u, CUT_TAIL_WITHOUT_HELPERS);
        return;
    }
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * S::kStageBytes + S::kOutStageBytes);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 2);    // the leader's A and B producer (used in the leader only)
            mbar_init(&empty_bar[s], 1);   // one commit, delivered to both CTAs
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full_bar[b], 1);
            mbar_init(&tmem_empty_bar[b], 8 * EPI_GROUPS);  // every epilogue warp of both CTAs (used in the leader only)
        }
        fence_mbar_init();
        tma_prefetch_desc(&p.tm_a);
        tma_prefetch_desc(&p.tm_b);
        if (p.tma_store) tma_prefetch_desc(&p.tm_out);
    }
    if (warp == 2) {
        tmem_alloc_pair(tmem_holder, 2 * kPairBlockN);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();      // both CTAs' barriers are initialised and both allocations are done
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    // Set-up is done without touching global memory; everything below reads operands or writes results that a kernel
    // earlier in the stream may produce or still use.
    griddep_wait();

    if (warp == 0 || warp == 3) {
        // ------------------------------------------------------------------ TMA producers (warp 0: A, warp 3: B)
        if (elect_one()) {
            const bool is_a = warp == 0;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            AFeed a_feed;
            BFeed<kPairBlockN / 2> b_feed;
            if (is_a) a_feed.setup(p); else b_feed.setup(p, p.tile_n / 2);
            const uint32_t my_bytes = is_a ? uint32_t(S::kABytes) : p.b_cta_bytes;
            const uint32_t dst_off = is_a ? 0u : uint32_t(S::kABytes);
            const uint32_t full0 = mapa_shared(smem_u32(&full_bar[0]), 0);   // the leader's full[0]
            PairSchedule<CUT> sched;
            sched.init(p, pair);
            TileCoord tc;
            uint32_t kind = WORK_TILE, slot = 0, above_slot = kNoSlot;
            while (ok && sched.next(p, pair, num_pairs, tc, kind, slot, above_slot)) {
                // first row (A) or column (B) this CTA stages
                if (is_a) a_feed.begin_tile(p, tc.m0 * 2 + rank * kBlockM, tc.batch, tc.kb_begin);
                else b_feed.begin_tile(p, tc.n0 * p.tile_n + rank * (p.tile_n / 2), tc.batch, tc.kb_begin);
                for (uint32_t kb = tc.kb_begin; kb < tc.kb_end; ++kb) {
                    if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, kWaitLimitNs)) {
                        atomicCAS(p.status, 0u, WAIT_PRODUCER_EMPTY);
                        ok = false;
                        break;
                    }
                    uint8_t* dst = smem + stage * S::kStageBytes + dst_off;
                    const uint32_t bar = full0 + stage * 8;
                    if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * my_bytes);   // this CTA's bytes and the partner's
                    if (is_a) a_feed.load<true>(p, dst, bar);
                    else b_feed.load<true>(p, dst, bar);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0 && elect_one()) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t mn_k_step = (kUmmaKBytes / p.elem_bytes) * kRowBytes;
            const uint32_t mn_lbo = p.block_k * kRowBytes;
            const uint32_t smem_base = smem_u32(smem);
            const uint64_t a_desc0 = p.a_mn_major ? make_smem_desc(smem_base, mn_lbo, 1024) : make_smem_desc(smem_base, 16, 1024);
            const uint64_t b_desc0 = p.b_mn_major ? make_smem_desc(smem_base + S::kABytes, mn_lbo, 1024)
                                                  : make_smem_desc(smem_base + S::kABytes, 16, 1024);
            const uint64_t a_step = (p.a_mn_major ? mn_k_step : uint32_t(kUmmaKBytes)) >> 4;
            const uint64_t b_step = (p.b_mn_major ? mn_k_step : uint32_t(kUmmaKBytes)) >> 4;
            constexpr uint64_t kStageUnits = S::kStageBytes >> 4;
            const uint32_t idesc = p.idesc;   // M = 256, N = tile_n
            PairSchedule<CUT> sched;
            sched.init(p, pair);
            TileCoord tc;
            uint32_t kind = WORK_TILE, slot = 0, above_slot = kNoSlot;
            while (ok && sched.next(p, pair, num_pairs, tc, kind, slot, above_slot)) {
                if (!mbar_wait_bounded(&tmem_empty_bar[acc], acc_phase ^ 1, kWaitLimitNs)) {
                    atomicCAS(p.status, 0u, WAIT_MMA_TMEM_EMPTY);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kPairBlockN;
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
                        umma_ss_pair<KIND>(d_tmem, a_desc + k * a_step, b_desc + k * b_step, idesc, accumulate);
                        accumulate = 1;
                    }
                    umma_commit_pair(&empty_bar[stage], 3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(&tmem_full_bar[acc], 3);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const uint32_t sub = warp & 3;           // tensor-memory lane window of this warp
        const uint32_t grp = (warp - 4) >> 2;    // which share of the columns
        constexpr int kGroupCols = kPairBlockN / EPI_GROUPS;
        uint32_t acc = 0, acc_phase = 0;
        const uint32_t out_elem = dtype_size(int(p.out_dtype));
        uint8_t* stage_out = smem + STAGES * S::kStageBytes + grp * (2 * kBlockM * kRowBytes);
        uint32_t store_buf = 0;
        const uint32_t leader_tmem_empty = mapa_shared(smem_u32(&tmem_empty_bar[0]), 0);
        PairSchedule<CUT> sched;
        sched.init(p, pair);
        TileCoord tc;
        uint32_t kind = WORK_TILE, slot = 0, above_slot = kNoSlot;
        while (sched.next(p, pair, num_pairs, tc, kind, slot, above_slot)) {
            bool ready = mbar_wait_bounded(&tmem_full_bar[acc], acc_phase, kWaitLimitNs);
            ready = __all_sync(0xffffffffu, ready);
            if (!ready) {
                atomicCAS(p.status, 0u, WAIT_EPILOGUE_TMEM_FULL);
                break;
            }
            tc_fence_after_sync();
            const uint32_t tmem_acc = tmem_base + acc * kPairBlockN + grp * kGroupCols + ((sub * 32) << 16);
            const uint32_t group_cols = p.tile_n > grp * kGroupCols ? min(uint32_t(kGroupCols), p.tile_n - grp * kGroupCols) : 0u;
            if constexpr (CUT) {
                // a cut tile: wait for the running sum of the pieces after this one (none after the last piece)
                const float* above = nullptr;
                if (kind != WORK_TILE && above_slot != kNoSlot) {
                    bool there = true;
                    if (lane == 0) there = flag_wait_bounded(p.sk_flags + (above_slot * 2 + rank) * kSkFlagsPerCta + (warp - 4), p.sk_gen, kSkWaitLimitNs);
                    there = __all_sync(0xffffffffu, there);
                    if (there) above = p.sk_ws + uint64_t(above_slot * 2 + rank) * kSkSlotFloats;
                    else atomicCAS(p.status, 0u, WAIT_STREAMK_PARTIAL);   // the tile is stored without the missing pieces; the call fails
                }
                if (kind == WORK_SK_WRITER) {
                    epilogue_partial(p.sk_ws + uint64_t(slot * 2 + rank) * kSkSlotFloats, above, grp * kGroupCols, group_cols, tmem_acc, sub * 32 + lane);
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence();
                        st_release_gpu(p.sk_flags + (slot * 2 + rank) * kSkFlagsPerCta + (warp - 4), p.sk_gen);
                    }
                } else {
                    const SkFix fix{above, above ? 1u : 0u, grp * kGroupCols};
                    epilogue_tile<true>(p, group_cols, tc.m0 * 2 + rank * kBlockM, tc.n0 * p.tile_n + grp * kGroupCols, tc.batch, tc.split, tmem_acc,
                                        stage_out, store_buf, sub, lane, out_elem, fix);
                }
            } else {
                epilogue_tile(p, group_cols, tc.m0 * 2 + rank * kBlockM, tc.n0 * p.tile_n + grp * kGroupCols, tc.batch, tc.split, tmem_acc,
                              stage_out, store_buf, sub, lane, out_elem);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tmem_empty + acc * 8);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (p.tma_store && lane == 0) tma_store_wait_all<0>();
    }

    // nobody may leave (or free tensor memory) while the partner can still signal this CTA's barriers or read its operands
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 2 * kPairBlockN);
    }
}

}  // namespace mmeb200
