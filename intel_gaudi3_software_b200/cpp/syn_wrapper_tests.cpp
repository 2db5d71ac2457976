// Exercises the Synapse-facing helpers (syn_cpu_calculator_b200.cpp) on a B200 the way Synapse's device tests
// use synapse/tests/utils/cpu_calculator.cpp: calculate* to produce a reference tensor, check* to judge a
// result buffer. Expected values come from plain double-precision loops over small-integer inputs, for which
// every product and partial sum is exact in fp32, so results must match bit for bit. Exit code 0 = all pass.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <stdexcept>
#include <vector>

#include "syn_cpu_calculator_b200.h"

static int g_failures = 0;
#define EXPECT(cond)                                                       \
    do {                                                                   \
        if (!(cond)) {                                                     \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
            ++g_failures;                                                  \
        }                                                                  \
    } while (0)

static uint16_t toBf16(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
static float fromBf16(uint16_t h)
{
    uint32_t u = uint32_t(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static synTensorDescriptor desc(synDataType t, std::vector<unsigned> sizes)
{
    unsigned s[SYN_MAX_TENSOR_DIM] = {1, 1, 1, 1, 1};
    for (size_t i = 0; i < sizes.size(); i++) s[i] = sizes[i];
    return synTensorDescriptor(t, unsigned(sizes.size()), s, nullptr);
}
static std::vector<uint16_t> smallInts(size_t n, int lo, int hi, unsigned seed)
{
    std::mt19937 rng(seed);
    std::uniform_int_distribution<int> d(lo, hi);
    std::vector<uint16_t> v(n);
    for (auto& e : v) e = toBf16(float(d(rng)));
    return v;
}

// Geometry of the convolution cases: x[C,W,H,B], w[K,C,S,R], y[K,Wo,Ho,B], 3x3 filter, pad 1, stride 1.
struct Conv
{
    unsigned C = 16, K = 24, W = 9, H = 7, B = 3, S = 3, R = 3;
    int pad = 1;
    unsigned Wo() const { return W + 2 * pad - S + 1; }
    unsigned Ho() const { return H + 2 * pad - R + 1; }
    synConvolution3DParams params(bool relu = false) const
    {
        synConvolution3DParams p;
        p.kernel[CONV_KERNEL_WIDTH] = S;
        p.kernel[CONV_KERNEL_HEIGHT] = R;
        p.padding[CONV_PAD_LEFT] = p.padding[CONV_PAD_RIGHT] = p.padding[CONV_PAD_TOP] = p.padding[CONV_PAD_BOTTOM] = pad;
        p.activation.reluEnable = relu;
        return p;
    }
    size_t xi(unsigned c, unsigned w, unsigned h, unsigned b) const { return ((size_t(b) * H + h) * W + w) * C + c; }
    size_t wi(unsigned k, unsigned c, unsigned s, unsigned r) const { return ((size_t(r) * S + s) * C + c) * K + k; }
    size_t yi(unsigned k, unsigned w, unsigned h, unsigned b) const { return ((size_t(b) * Ho() + h) * Wo() + w) * K + k; }
};

static void naiveFwd(const Conv& g, const std::vector<uint16_t>& x, const std::vector<uint16_t>& w, std::vector<double>& y)
{
    y.assign(size_t(g.K) * g.Wo() * g.Ho() * g.B, 0.0);
    for (unsigned b = 0; b < g.B; b++)
        for (unsigned ho = 0; ho < g.Ho(); ho++)
            for (unsigned wo = 0; wo < g.Wo(); wo++)
                for (unsigned r = 0; r < g.R; r++)
                    for (unsigned s = 0; s < g.S; s++)
                    {
                        const int hi = int(ho) + int(r) - g.pad, wi = int(wo) + int(s) - g.pad;
                        if (hi < 0 || wi < 0 || hi >= int(g.H) || wi >= int(g.W)) continue;
                        for (unsigned c = 0; c < g.C; c++)
                            for (unsigned k = 0; k < g.K; k++)
                                y[g.yi(k, wo, ho, b)] += double(fromBf16(x[g.xi(c, wi, hi, b)])) * fromBf16(w[g.wi(k, c, s, r)]);
                    }
}
static void naiveDedx(const Conv& g, const std::vector<uint16_t>& dy, const std::vector<uint16_t>& w, std::vector<double>& dx)
{
    dx.assign(size_t(g.C) * g.W * g.H * g.B, 0.0);
    for (unsigned b = 0; b < g.B; b++)
        for (unsigned ho = 0; ho < g.Ho(); ho++)
            for (unsigned wo = 0; wo < g.Wo(); wo++)
                for (unsigned r = 0; r < g.R; r++)
                    for (unsigned s = 0; s < g.S; s++)
                    {
                        const int hi = int(ho) + int(r) - g.pad, wi = int(wo) + int(s) - g.pad;
                        if (hi < 0 || wi < 0 || hi >= int(g.H) || wi >= int(g.W)) continue;
                        for (unsigned c = 0; c < g.C; c++)
                            for (unsigned k = 0; k < g.K; k++)
                                dx[g.xi(c, wi, hi, b)] += double(fromBf16(dy[g.yi(k, wo, ho, b)])) * fromBf16(w[g.wi(k, c, s, r)]);
                    }
}
static void naiveDedw(const Conv& g, const std::vector<uint16_t>& x, const std::vector<uint16_t>& dy, std::vector<double>& dw)
{
    dw.assign(size_t(g.K) * g.C * g.S * g.R, 0.0);
    for (unsigned b = 0; b < g.B; b++)
        for (unsigned ho = 0; ho < g.Ho(); ho++)
            for (unsigned wo = 0; wo < g.Wo(); wo++)
                for (unsigned r = 0; r < g.R; r++)
                    for (unsigned s = 0; s < g.S; s++)
                    {
                        const int hi = int(ho) + int(r) - g.pad, wi = int(wo) + int(s) - g.pad;
                        if (hi < 0 || wi < 0 || hi >= int(g.H) || wi >= int(g.W)) continue;
                        for (unsigned c = 0; c < g.C; c++)
                            for (unsigned k = 0; k < g.K; k++)
                                dw[g.wi(k, c, s, r)] += double(fromBf16(x[g.xi(c, wi, hi, b)])) * fromBf16(dy[g.yi(k, wo, ho, b)]);
                    }
}

static void convolutions()
{
    Conv g;
    const auto x = smallInts(size_t(g.C) * g.W * g.H * g.B, -3, 3, 1), w = smallInts(size_t(g.K) * g.C * g.S * g.R, -2, 2, 2);
    const auto dy = smallInts(size_t(g.K) * g.Wo() * g.Ho() * g.B, -2, 2, 3);
    const synTensorDescriptor xd = desc(syn_type_bf16, {g.C, g.W, g.H, g.B}), wd = desc(syn_type_bf16, {g.K, g.C, g.S, g.R}),
                              yd = desc(syn_type_bf16, {g.K, g.Wo(), g.Ho(), g.B}), wd32 = desc(syn_type_float, {g.K, g.C, g.S, g.R});
    std::vector<double> want;
    CoordArray idx;

    // forward, with and without ReLU
    for (bool relu : {false, true})
    {
        std::vector<uint16_t> y(dy.size(), 0xDEAD);
        calculateFwdConvolution(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), g.params(relu), synDeviceGaudi3);
        naiveFwd(g, x, w, want);
        size_t bad = 0;
        for (size_t i = 0; i < y.size(); i++) bad += y[i] != toBf16(float(relu && want[i] < 0 ? 0.0 : want[i]));
        EXPECT(bad == 0);
        if (!relu)
        {
            EXPECT(checkFwdConvolution(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), g.params(), idx, synDeviceGaudi3));
            EXPECT(idx[0] == 0 && idx[1] == 0 && idx[2] == 0 && idx[3] == 0);
            // spoil one element: the check must fail there and report the reference value
            const size_t victim = g.yi(5, 2, 3, 1);
            const uint16_t keep = y[victim];
            y[victim] = toBf16(fromBf16(keep) + 64.0f);
            float expected = 0;
            EXPECT(!checkMmeOp(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), g.params(), REFERENCE_OP_FWD, idx,
                               synDeviceGaudi3, &expected));
            EXPECT(idx[0] == 5 && idx[1] == 2 && idx[2] == 3 && idx[3] == 1);
            uint32_t raw;
            std::memcpy(&raw, &expected, 4);
            EXPECT(uint16_t(raw) == keep);
        }
    }
    // dedx into bf16
    {
        std::vector<uint16_t> dx(x.size(), 0xDEAD);
        calculateDEDX(yd, (char*) dy.data(), wd, (char*) w.data(), xd, (char*) dx.data(), g.params(), synDeviceGaudi3);
        naiveDedx(g, dy, w, want);
        size_t bad = 0;
        for (size_t i = 0; i < dx.size(); i++) bad += dx[i] != toBf16(float(want[i]));
        EXPECT(bad == 0);
        EXPECT(checkDEDX(yd, (char*) dy.data(), wd, (char*) w.data(), xd, (char*) dx.data(), g.params(), idx, synDeviceGaudi3));
    }
    // dedw into fp32
    {
        std::vector<float> dw(w.size(), -1.0f);
        calculateDEDW(yd, (char*) dy.data(), xd, (char*) x.data(), wd32, (char*) dw.data(), g.params(), synDeviceGaudi3);
        naiveDedw(g, x, dy, want);
        size_t bad = 0;
        for (size_t i = 0; i < dw.size(); i++) bad += dw[i] != float(want[i]);
        EXPECT(bad == 0);
        EXPECT(checkDEDW(yd, (char*) dy.data(), xd, (char*) x.data(), wd32, (char*) dw.data(), g.params(), idx, synDeviceGaudi3));
        dw[7] += 3.0f;
        EXPECT(!checkDEDW(yd, (char*) dy.data(), xd, (char*) x.data(), wd32, (char*) dw.data(), g.params(), idx, synDeviceGaudi3));
        EXPECT(idx[0] == 7 && idx[1] == 0);
        // the statistical rule: one spoiled element out of thousands keeps the correlation, a scrambled result does not
        EXPECT(checkDEDW(yd, (char*) dy.data(), xd, (char*) x.data(), wd32, (char*) dw.data(), g.params(), idx, synDeviceGaudi3, true));
        std::vector<float> scrambled(dw.rbegin(), dw.rend());
        EXPECT(!checkDEDW(yd, (char*) dy.data(), xd, (char*) x.data(), wd32, (char*) scrambled.data(), g.params(), idx, synDeviceGaudi3, true));
        std::vector<float> halved(dw);
        for (auto& v : halved) v *= 0.5f;   // perfectly correlated, but the L2 norms differ by a factor of two
        EXPECT(!checkDEDW(yd, (char*) dy.data(), xd, (char*) x.data(), wd32, (char*) halved.data(), g.params(), idx, synDeviceGaudi3, true));
    }
}

static void gemms()
{
    const unsigned M = 37, N = 40, Kd = 72, batch = 3;
    CoordArray idx;
    // bf16, batched, ab: x[K, M, b] . w[N, K, b] -> y[N, M, b]
    {
        const auto x = smallInts(size_t(Kd) * M * batch, -3, 3, 4), w = smallInts(size_t(N) * Kd * batch, -3, 3, 5);
        std::vector<uint16_t> y(size_t(N) * M * batch, 0xDEAD);
        const synTensorDescriptor xd = desc(syn_type_bf16, {Kd, M, batch}), wd = desc(syn_type_bf16, {N, Kd, batch}),
                                  yd = desc(syn_type_bf16, {N, M, batch});
        calculateGemm(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), synGEMMParams(), REFERENCE_OP_AB, synDeviceGaudi3);
        size_t bad = 0;
        for (unsigned b = 0; b < batch; b++)
            for (unsigned m = 0; m < M; m++)
                for (unsigned n = 0; n < N; n++)
                {
                    double s = 0;
                    for (unsigned k = 0; k < Kd; k++)
                        s += double(fromBf16(x[(size_t(b) * M + m) * Kd + k])) * fromBf16(w[(size_t(b) * Kd + k) * N + n]);
                    bad += y[(size_t(b) * M + m) * N + n] != toBf16(float(s));
                }
        EXPECT(bad == 0);
        float expected = 0;
        EXPECT(checkBatchGemmOp(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), REFERENCE_OP_AB, idx, &expected,
                                synDeviceGaudi3));
        y[(size_t(2) * M + 11) * N + 13] ^= 0x4000;
        EXPECT(!checkBatchGemmOp(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), REFERENCE_OP_AB, idx, &expected,
                                 synDeviceGaudi3));
        EXPECT(idx[0] == 13 && idx[1] == 11 && idx[2] == 2);
    }
    // fp8_143 with the default exponent bias (7): codes of small integers, abt: x[K, M] . w[K, N]^T -> fp32
    {
        // 1-4-3, bias 7: 0x38 = 1.0, 0x40 = 2.0, 0x44 = 3.0, sign bit 0x80
        const uint8_t code[7] = {0xC4, 0xC0, 0xB8, 0x00, 0x38, 0x40, 0x44};
        const float value[7] = {-3, -2, -1, 0, 1, 2, 3};
        std::mt19937 rng(6);
        std::vector<uint8_t> x(size_t(Kd) * M), w(size_t(Kd) * N);
        std::vector<float> xf(x.size()), wf(w.size());
        for (size_t i = 0; i < x.size(); i++) { const unsigned j = rng() % 7; x[i] = code[j]; xf[i] = value[j]; }
        for (size_t i = 0; i < w.size(); i++) { const unsigned j = rng() % 7; w[i] = code[j]; wf[i] = value[j]; }
        std::vector<float> y(size_t(N) * M, -1.0f);
        const synTensorDescriptor xd = desc(syn_type_fp8_143, {Kd, M}), wd = desc(syn_type_fp8_143, {Kd, N}), yd = desc(syn_type_float, {N, M});
        calculateGemm(xd, (char*) x.data(), wd, (char*) w.data(), yd, (char*) y.data(), synGEMMParams(), REFERENCE_OP_ABT, synDeviceGaudi3);
        size_t bad = 0;
        for (unsigned m = 0; m < M; m++)
            for (unsigned n = 0; n < N; n++)
            {
                double s = 0;
                for (unsigned k = 0; k < Kd; k++) s += double(xf[size_t(m) * Kd + k]) * wf[size_t(n) * Kd + k];
                bad += y[size_t(m) * N + n] != float(s);
            }
        EXPECT(bad == 0);
    }
    // masked bgemm: y = x.w + xMask.wMask
    {
        const unsigned Km = 8;
        const auto x = smallInts(size_t(Kd) * M, -3, 3, 7), w = smallInts(size_t(N) * Kd, -3, 3, 8);
        const auto xm = smallInts(size_t(Km) * M, 0, 1, 9), wm = smallInts(size_t(N) * Km, -4, 0, 10);
        std::vector<uint16_t> y(size_t(N) * M);
        for (unsigned m = 0; m < M; m++)
            for (unsigned n = 0; n < N; n++)
            {
                double s = 0;
                for (unsigned k = 0; k < Kd; k++) s += double(fromBf16(x[size_t(m) * Kd + k])) * fromBf16(w[size_t(k) * N + n]);
                for (unsigned k = 0; k < Km; k++) s += double(fromBf16(xm[size_t(m) * Km + k])) * fromBf16(wm[size_t(k) * N + n]);
                y[size_t(m) * N + n] = toBf16(float(s));
            }
        const synTensorDescriptor xd = desc(syn_type_bf16, {Kd, M}), wd = desc(syn_type_bf16, {N, Kd}), xmd = desc(syn_type_bf16, {Km, M}),
                                  wmd = desc(syn_type_bf16, {N, Km}), yd = desc(syn_type_bf16, {N, M});
        float expected = 0;
        EXPECT(checkMaskedBatchGemmOp(xd, (char*) x.data(), wd, (char*) w.data(), xmd, (char*) xm.data(), wmd, (char*) wm.data(), yd,
                                      (char*) y.data(), REFERENCE_OP_AB, idx, &expected, synDeviceGaudi3));
        y[size_t(3) * N + 1] ^= 0x4000;
        EXPECT(!checkMaskedBatchGemmOp(xd, (char*) x.data(), wd, (char*) w.data(), xmd, (char*) xm.data(), wmd, (char*) wm.data(), yd,
                                       (char*) y.data(), REFERENCE_OP_AB, idx, &expected, synDeviceGaudi3));
        EXPECT(idx[0] == 1 && idx[1] == 3);
    }
}

static void hostHelpers()
{
    CoordArray idx;
    const synTensorDescriptor d = desc(syn_type_float, {4, 3});
    std::vector<float> a(12, 1.0f), b(12, 1.0f), out(12);
    b[5] = 1.001f;   // inside 1e-7 + 0.0015 * 1
    EXPECT(checkResults(d, (char*) a.data(), (char*) b.data(), idx));
    b[9] = 1.01f;
    EXPECT(!checkResults(d, (char*) a.data(), (char*) b.data(), idx));
    EXPECT(idx[0] == 1 && idx[1] == 2);
    a[9] = b[9] = NAN;
    EXPECT(checkResults(d, (char*) a.data(), (char*) b.data(), idx));
    a[9] = 2.5f; b[9] = -0.25f;
    calculateAdd(d, (char*) a.data(), (char*) b.data(), (char*) out.data());
    EXPECT(out[9] == 2.25f && out[0] == 2.0f);
    const synTensorDescriptor dh = desc(syn_type_bf16, {4});
    const uint16_t ha[4] = {toBf16(1.0f), toBf16(256.0f), toBf16(-3.0f), toBf16(0.5f)}, hb[4] = {toBf16(2.0f), toBf16(1.0f), toBf16(3.0f), toBf16(0.25f)};
    uint16_t ho[4];
    calculateAdd(dh, (char*) ha, (char*) hb, (char*) ho);
    EXPECT(ho[0] == toBf16(3.0f) && ho[1] == toBf16(256.0f) && ho[2] == toBf16(0.0f) && ho[3] == toBf16(0.75f));   // 257 rounds to even
    const TSize sizes[4] = {4, 3, 1, 1};
    CoordArray at = {1, 2, 0, 0, 0};
    EXPECT(getIndexValue(sizes, at, syn_type_float, a.data()) == 2.5f);
}

int main()
{
    try
    {
        convolutions();
        gemms();
        hostHelpers();
    }
    catch (const std::exception& e)
    {
        std::printf("FAILED with exception: %s\n", e.what());
        return 2;
    }
    if (g_failures == 0) std::printf("all passed\n");
    return g_failures ? 1 : 0;
}
