// TEST INFRASTRUCTURE: compiles the product's device conversion functions (csrc/numerics.cuh, which
// are __host__ __device__) for the host, so that their bit patterns can be compared against the CPU
// oracle on a machine without a GPU. Nothing in the product links or calls this file.
#include <cstddef>
#include <cstdint>

#include "numerics.cuh"
#include "gaudi3_exact.cuh"
#include "schedule.cuh"

using namespace mmeb200;

// the epilogue's straight-line casts (slow: reserved, always 0)
template <int RM>
static void cast_flat(const uint32_t* in, uint8_t* out, uint8_t* slow, size_t n, int out_dtype, int exp_width, int bias, int mode, int clip,
                      int clip_inf_in, int ftz, const uint32_t* rnd)
{
    for (size_t i = 0; i < n; i++) {
        if (out_dtype == DT_BF16) {
            const uint32_t v = f32_to_bf16_flat<RM>(in[i], rnd[i], clip, ftz, clip_inf_in);
            out[2 * i] = uint8_t(v);
            out[2 * i + 1] = uint8_t(v >> 8);
            slow[i] = 0;
        } else {
            out[i] = uint8_t(f32_to_fp8_flat<RM>(in[i], exp_width, bias, rnd[i], mode, clip, clip_inf_in));
            slow[i] = 0;
        }
    }
}
extern "C" {
void hc_fp8_decode(const uint8_t* in, uint32_t* out, size_t n, int exp_width, int bias, int mode)
{
    for (size_t i = 0; i < n; i++) out[i] = fp8_decode(in[i], exp_width, bias, mode);
}
void hc_cast(const uint32_t* in, uint8_t* out, size_t n, int out_dtype, int exp_width, int bias, int mode, int rm, int relu, int clip,
             int clip_inf_in, int ftz, int sftz, const uint32_t* rnd)
{
    CastSpec c{out_dtype, exp_width, bias, mode, rm, relu, clip, clip_inf_in, ftz, sftz};
    const int es = dtype_size(out_dtype);
    for (size_t i = 0; i < n; i++) {
        uint32_t b = in[i];
        if (relu) b = relu_bits(b);
        const uint32_t v = cast_from_f32(b, c, rnd ? rnd[i] : 0);
        for (int k = 0; k < es; k++) out[i * es + k] = uint8_t(v >> (8 * k));
    }
}
int hc_cast_flat(const uint32_t* in, uint8_t* out, uint8_t* slow, size_t n, int out_dtype, int exp_width, int bias, int mode, int rm, int clip,
                 int clip_inf_in, int ftz, const uint32_t* rnd)
{
    switch (rm) {
#define FLAT_CASE(R) case R: cast_flat<R>(in, out, slow, n, out_dtype, exp_width, bias, mode, clip, clip_inf_in, ftz, rnd); return 0;
        FLAT_CASE(RM_NE) FLAT_CASE(RM_Z) FLAT_CASE(RM_UP) FLAT_CASE(RM_DOWN) FLAT_CASE(RM_SR) FLAT_CASE(RM_HAZ) FLAT_CASE(RM_SR_NE_DNORM)
#undef FLAT_CASE
    }
    return -1;
}
// Host model of the hardware fp8 path (f32x4_to_fp8_hw): the product's rescale, thresholds and constant codes (fp8_hw_cast,
// fp8_hw_fix) around a model of the saturating hardware conversion -- round-to-nearest-even into the hardware format's own
// bias and Inf/NaN convention with everything above the largest finite value clamped to it.
int hc_cast_fp8_hw_model(const uint32_t* in, uint8_t* out, size_t n, int out_dtype, int exp_width, int bias, int mode, int clip, int clip_inf_in)
{
    CastSpec c{out_dtype, exp_width, bias, mode, RM_NE, 0, clip, clip_inf_in, 0, 0};
    if (!cast_is_fp8_hw(c)) return -1;
    const Fp8HwCast h = fp8_hw_cast(c);
    const bool e4m3 = out_dtype == DT_FP8_143;
    for (size_t i = 0; i < n; i++) {
        const float x = bits_as_float(in[i]);
        const float f = x * h.scale;
        uint32_t fb;
        memcpy(&fb, &f, 4);
        const uint32_t fix = fp8_hw_fix(x, f, h);
        const uint32_t hw = e4m3 ? f32_to_fp8(fb, 4, 7, RM_NE, 0, false, true, true, false, 2) : f32_to_fp8(fb, 5, 15, RM_NE, 0, false, true, true, false, 0);
        out[i] = uint8_t(fix != 0x100u ? fix : hw);
    }
    return 0;
}
void hc_compare(const uint8_t* a, const uint8_t* b, uint8_t* equal, size_t n, int dtype, int bias, int mode, unsigned cd)
{
    const CompareSpec c = make_compare_spec(dtype, bias, mode, cd);
    const int es = dtype_size(dtype);
    for (size_t i = 0; i < n; i++) {
        uint32_t ra = 0, rb = 0;
        for (int k = 0; k < es; k++) { ra |= uint32_t(a[i * es + k]) << (8 * k); rb |= uint32_t(b[i * es + k]) << (8 * k); }
        equal[i] = compare_elements(ra, rb, c) ? 1 : 0;
    }
}
void hc_bf16_rmw(uint16_t* mem, const uint16_t* in, size_t n, int op, int rm, int clip)
{
    for (size_t i = 0; i < n; i++) mem[i] = uint16_t(bf16_rmw(mem[i], in[i], op, rm, clip != 0));
}
void hc_fp8_152_rmw(uint8_t* mem, const uint8_t* in, size_t n, int op, int rm, int clip)
{
    for (size_t i = 0; i < n; i++) mem[i] = uint8_t(fp8_152_rmw(mem[i], in[i], op, rm, clip != 0));
}
// dot product of n decoded fp32 bit patterns in the reference's block order (blocks of eight, zero-padded tail)
uint32_t hc_g3_dot(const uint32_t* a, const uint32_t* b, size_t n)
{
    uint32_t c = 0;
    for (size_t k = 0; k < n; k += 8) {
        uint32_t ta[8], tb[8];
        for (size_t i = 0; i < 8; i++) { ta[i] = k + i < n ? a[k + i] : 0; tb[i] = k + i < n ? b[k + i] : 0; }
        c = g3_tree8(ta, tb, c);
    }
    return c;
}
uint32_t hc_g3_dot_fp32(const uint32_t* a, const uint32_t* b, size_t n)
{
    uint32_t c = 0;
    for (size_t k = 0; k < n; k++) c = g3_fp32_mac(a[k], b[k], c);
    return c;
}
uint32_t hc_g3_dot_tf32(const uint32_t* a, const uint32_t* b, size_t n)
{
    uint32_t c = 0;
    for (size_t k = 0; k < n; k += 2)
        c = g3_tf32_mac2(tf32_rne_bits(a[k]), tf32_rne_bits(b[k]), k + 1 < n ? tf32_rne_bits(a[k + 1]) : 0, k + 1 < n ? tf32_rne_bits(b[k + 1]) : 0, c);
    return c;
}
int hc_fp8_foreign(uint32_t code, int exp_width, int mode) { return fp8_code_is_foreign(code, exp_width, mode); }
uint32_t hc_lfsr(uint32_t v, uint32_t poly) { return lfsr32_step(v, poly); }
uint32_t hc_philox(uint64_t seed, uint64_t offset, uint64_t index) { return philox_word(seed, offset, index); }
uint32_t hc_philox_half(uint64_t seed, uint64_t offset, uint64_t index) { return philox_half(seed, offset, index); }
void hc_philox_halves(uint64_t seed, uint64_t offset, uint64_t index8, uint32_t* w8, uint32_t* w4a, uint32_t* w4b)
{
    uint32_t a[8], b[4], c[4];
    philox_halves8(seed, offset, index8, a);
    philox_halves4(seed, offset, index8, b);
    philox_halves4(seed, offset, index8 + 4, c);
    for (int i = 0; i < 8; i++) w8[i] = a[i];
    for (int i = 0; i < 4; i++) { w4a[i] = b[i]; w4b[i] = c[i]; }
}
// Stochastic rounding of groups of eight with their raw Philox blocks (blocks: 4 words per group): the addition form
// (sr_bf16_group8 / sr_fp8_group8) into `fast`, the straight-line cast element by element into `flat`.
void hc_sr_groups(const uint32_t* in, const uint32_t* blocks, size_t groups, int out_dtype, int exp_width, int bias, int mode, int clip,
                  int clip_inf_in, int canon_nan, uint8_t* fast, uint8_t* flat)
{
    const Fp8SrSpec sp = fp8_sr_spec(exp_width, bias, mode);
    for (size_t g = 0; g < groups; g++) {
        const uint32_t* x = in + 8 * g;
        const uint32_t c[4] = {blocks[4 * g], blocks[4 * g + 1], blocks[4 * g + 2], blocks[4 * g + 3]};
        if (out_dtype == DT_BF16) {
            uint32_t w[4];
            sr_bf16_group8(x, c, clip, clip_inf_in, w);
            for (int e = 0; e < 8; e++) {
                const uint32_t v = (w[e >> 1] >> (16 * (e & 1))) & 0xFFFFu;
                const uint32_t r = f32_to_bf16_flat<RM_SR>(x[e], philox_block8_word(c, e), clip, false, clip_inf_in);
                fast[16 * g + 2 * e] = uint8_t(v); fast[16 * g + 2 * e + 1] = uint8_t(v >> 8);
                flat[16 * g + 2 * e] = uint8_t(r); flat[16 * g + 2 * e + 1] = uint8_t(r >> 8);
            }
        } else {
            uint32_t w[2];
            sr_fp8_group8(x, c, sp, exp_width, bias, mode, clip, clip_inf_in, canon_nan, w);
            for (int e = 0; e < 8; e++) {
                const uint32_t xin = (canon_nan && f32_is_nan(x[e])) ? kF32CanonNan : x[e];
                fast[8 * g + e] = uint8_t(w[e >> 2] >> (8 * (e & 3)));
                flat[8 * g + e] = uint8_t(f32_to_fp8_flat<RM_SR>(xin, exp_width, bias, philox_block8_word(c, e), mode, clip, clip_inf_in));
            }
        }
    }
}
void hc_philox_block8(uint64_t seed, uint64_t offset, uint64_t index8, uint32_t* c4, uint32_t* words8)
{
    uint32_t c[4];
    philox_block8(seed, offset, index8, c);
    for (int i = 0; i < 4; i++) c4[i] = c[i];
    for (int e = 0; e < 8; e++) words8[e] = philox_block8_word(c, e);
}
// The schedule the CTA-pair kernel walks (schedule.cuh), on the host: the planner's cut for `tiles` tiles of nkb k blocks on
// `units` pairs, and the work items of one pair. An item is 8 words: m0, n0, batch, kb_begin, kb_end, kind, slot, above.
struct HostSchedParams {
    uint32_t m_tiles, n_tiles, batches, split_k, raster_gm, num_k_blocks, sk_tiles, sk_head, sk_piece, sk_pieces;
};
uint64_t hc_plan_cut_tail(uint64_t rem, uint64_t units, uint32_t nkb, int any, uint32_t* head_piece_pieces)
{
    const CutPlan c = plan_cut_tail(rem, units, nkb, any != 0);
    head_piece_pieces[0] = c.head; head_piece_pieces[1] = c.piece; head_piece_pieces[2] = c.pieces;
    return c.cost;
}
uint32_t hc_plan_raster_group(uint64_t tile_rows, uint64_t K, uint32_t elem) { return plan_raster_group(tile_rows, K, elem); }
int hc_schedule_items(const uint32_t* params10, int cut, uint32_t pair, uint32_t num_pairs, uint32_t* items, int max_items)
{
    HostSchedParams p;
    memcpy(&p, params10, sizeof p);
    TileCoord tc{};
    uint32_t kind = WORK_TILE, slot = 0, above = kNoSlot;
    int n = 0;
    auto put = [&]() {
        if (n < max_items) {
            uint32_t* o = items + 8 * n;
            o[0] = tc.m0; o[1] = tc.n0; o[2] = tc.batch; o[3] = tc.kb_begin; o[4] = tc.kb_end; o[5] = kind; o[6] = slot; o[7] = above;
        }
        ++n;
    };
    if (cut) {
        PairSchedule<true> s;
        s.init(p, pair);
        while (s.next(p, pair, num_pairs, tc, kind, slot, above)) put();
    } else {
        PairSchedule<false> s;
        s.init(p, pair);
        kind = WORK_TILE; slot = 0; above = kNoSlot;
        while (s.next(p, pair, num_pairs, tc, kind, slot, above)) put();
    }
    return n;
}
void hc_philox_block(uint32_t* c, uint32_t k0, uint32_t k1)
{
    uint32_t s[4] = {c[0], c[1], c[2], c[3]};
    philox4x32_10(s, k0, k1);
    for (int i = 0; i < 4; i++) c[i] = s[i];
}
}
