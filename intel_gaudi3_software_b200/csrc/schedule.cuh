// Which tile, and which k blocks of it, a CTA (or CTA pair) of the persistent tcgen05 GEMM kernels works on next, and the
// planner's arithmetic for the cut tail and the raster. Everything here is plain integer code over a parameter block
// (GemmParams on the device; any struct with the same field names on the host), so the host tests walk the same schedule
// the kernels walk.
#pragma once
#include <stdint.h>

#include "numerics.cuh"   // MME_HD

namespace mmeb200 {

constexpr int kBlockM = 128;   // rows of an output tile per CTA

MME_HD uint32_t sched_min(uint32_t a, uint32_t b) { return a < b ? a : b; }

struct TileCoord {
    uint32_t m0, n0, batch, kb_begin, kb_end, split;
};

template <class P>
MME_HD TileCoord decode_tile(const P& p, uint32_t t) {
    TileCoord c;
    c.split = t % p.split_k;
    t /= p.split_k;
    const uint32_t per_batch = p.m_tiles * p.n_tiles;
    c.batch = t / per_batch;
    const uint32_t r = t % per_batch;
    const uint32_t GM = p.raster_gm;
    const uint32_t group_span = GM * p.n_tiles;
    const uint32_t first_m = (r / group_span) * GM;
    const uint32_t gsz = sched_min(GM, p.m_tiles - first_m);
    const uint32_t in_group = r % group_span;
    c.m0 = (first_m + in_group % gsz) * kBlockM;
    c.n0 = (in_group / gsz);  // tile index; scaled by the caller's BLOCK_N
    const uint32_t per_split = (p.num_k_blocks + p.split_k - 1) / p.split_k;
    c.kb_begin = c.split * per_split;
    c.kb_end = sched_min(p.num_k_blocks, c.kb_begin + per_split);
    return c;
}

// The work items of one pair, in the order every role of both CTAs walks them. With a cut tail (p.sk_tiles != 0): pair
// t < sk_tiles starts with the head of cut tile t; pair sk_tiles + h takes the pieces j = h, h + helpers, ... where piece j is
// piece sk_pieces - j / sk_tiles (counted from 1, so a tile's later pieces come first) of cut tile j % sk_tiles. Then, cut
// tail or not, the whole tiles t = pair, pair + pairs, ... of the tiles before the cut ones.
enum : uint32_t { WORK_TILE = 0, WORK_SK_WRITER = 1, WORK_SK_OWNER = 2 };
constexpr uint32_t kNoSlot = 0xFFFFFFFFu;
// What next() hands out beside the tile's coordinates (cut-tail kernel only): kind (WORK_*), slot (WORK_SK_WRITER: where
// this piece's running sum goes) and above (cut tiles: the slot with the running sum of the pieces after this one, or
// kNoSlot). They are separate scalars, not a struct: every role keeps them in registers across its k loop.
template <bool CUT>
struct PairSchedule {
    uint32_t j;              // next piece of a helper pair (past the end for the others)
    uint32_t t;              // next whole tile
    bool head;               // the head of cut tile `pair` is still to do
    uint32_t total;          // work items the planner counted: (tile, split) pairs, the cut tiles included
    template <class P>
    MME_HD void init(const P& p, uint32_t pair) {
        total = p.m_tiles * p.n_tiles * p.batches * p.split_k;
        t = pair;
        head = CUT && pair < p.sk_tiles;
        j = (CUT && pair >= p.sk_tiles) ? pair - p.sk_tiles : kNoSlot;
    }
    template <class P>
    MME_HD bool next(const P& p, uint32_t pair, uint32_t num_pairs, TileCoord& tc, uint32_t& kind, uint32_t& slot, uint32_t& above) {
        // the kernel without a cut tail: whole tiles only, and nothing else in the loop that every role runs between two tiles
        // (recomputing the tile count there and three dead stores cost 3-7 % on the bf16 GEMM and the convolutions)
        if constexpr (!CUT) {
            if (t >= total) return false;
            tc = decode_tile(p, t);
            t += num_pairs;
            return true;
        }
        kind = WORK_TILE;
        slot = 0;
        above = kNoSlot;
        const uint32_t whole_tiles = total - p.sk_tiles;
        if (head) {
            head = false;
            tc = decode_tile(p, whole_tiles + pair);
            tc.kb_end = p.sk_head;
            kind = WORK_SK_OWNER;
            above = pair * p.sk_pieces;
            return true;
        }
        if (j < p.sk_tiles * p.sk_pieces) {
            const uint32_t round = j / p.sk_tiles, tile = j - round * p.sk_tiles;
            const uint32_t piece = p.sk_pieces - round;
            tc = decode_tile(p, whole_tiles + tile);
            tc.kb_begin = p.sk_head + (piece - 1) * p.sk_piece;
            tc.kb_end = sched_min(p.num_k_blocks, tc.kb_begin + p.sk_piece);
            kind = WORK_SK_WRITER;
            slot = tile * p.sk_pieces + piece - 1;
            if (piece < p.sk_pieces) above = slot + 1;
            j += num_pairs - p.sk_tiles;
            return true;
        }
        if (t < whole_tiles) {
            tc = decode_tile(p, t);
            t += num_pairs;
            return true;
        }
        return false;
    }
};

// ---------------------------------------------------------------------------------------------
// Planner arithmetic (host)
// ---------------------------------------------------------------------------------------------
// Cut tail: `rem` tiles of num_k_blocks = nkb k blocks each are left over after the whole waves of `units` pairs. Each is cut
// into a head of `head` k blocks and `pieces` pieces of `piece` k blocks; rem pairs take the heads, the other units - rem
// share the pieces. The plan is the one that finishes earliest by a cost in k blocks: a piece's pair is busy for the piece's
// k blocks or, if longer, for the epilogue that writes its sums (about sixteen k blocks' time, measured), and four k blocks
// stand for the extra epilogue work. head == 0: no cut (none exists, or none beats the nkb k blocks of a whole tile unless
// `any` asks for the first one that exists). At most 224 slots.
struct CutPlan {
    uint32_t head, piece, pieces;
    uint64_t cost;
};
inline CutPlan plan_cut_tail(uint64_t rem, uint64_t units, uint32_t nkb, bool any) {
    CutPlan best{0u, 0u, 0u, nkb};
    if (rem == 0 || units <= rem) return best;
    const uint64_t helpers = units - rem;
    uint32_t first = uint32_t((rem * nkb + units - 1) / units);
    if (first < 4) first = 4;
    for (uint32_t head = first; head < nkb; ++head) {
        const uint32_t rest = nkb - head;
        const uint32_t pieces = (rest + head - 1) / head, piece = (rest + pieces - 1) / pieces;
        if (rem * pieces > 224 || piece < 2) break;
        const uint64_t rounds = (rem * pieces + helpers - 1) / helpers;
        const uint64_t helper_time = rounds * (piece > 16u ? piece : 16u);
        const uint64_t cost = (head > helper_time ? head : helper_time) + 4;
        if (cost < best.cost || (any && best.head == 0)) {
            best.head = head; best.piece = piece; best.pieces = pieces;
            best.cost = cost < nkb ? cost : nkb;
        }
        if (rounds * piece <= head) break;   // longer heads only finish later
    }
    return best;
}
// Raster group (m tiles per group): the A panel of a group (its m tiles x all of K) should stay in L2 while the group's
// n tiles stream B past it. About 32 MiB does (the L2's two halves each keep their own copy of what both read): 16 m tiles of
// 256 rows for fp8 at K = 8192, 8 for bf16 (measured there: 8 is 3 % faster than 16, burst and sustained; for fp8 16 is 2 %
// faster than 8). 32-bit operands keep 16 (their K-major copies are three times as long for fp32; 4 measured 1 % slower).
inline uint32_t plan_raster_group(uint64_t tile_rows, uint64_t K, uint32_t elem_bytes) {
    const uint64_t tile_bytes = tile_rows * K * elem_bytes;
    return (elem_bytes <= 2 && 16 * tile_bytes > (uint64_t(32) << 20)) ? 8u : 16u;
}

}  // namespace mmeb200
