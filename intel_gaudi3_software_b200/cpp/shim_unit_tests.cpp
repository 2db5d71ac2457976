// The calculator cases of the reference's unit tests (mme/tests/unit_tests/mme_unit_test.cpp:67-172,
// 425-465, 498-575), restated without gtest and run against the drop-in calculator
// (mme_reference_b200.cpp) on a B200. Exit code 0 = all cases pass.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "mme_reference.h"
#include "data_types/non_standard_dtypes.h"
#include "sim_tensor.h"
#include "tensor_comparator.h"

using namespace MmeCommon;

static int g_failures = 0;
#define EXPECT(cond)                                                       \
    do {                                                                   \
        if (!(cond)) {                                                     \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
            ++g_failures;                                                  \
        }                                                                  \
    } while (0)

static MmeSimTensor createSimTensor(SizeArray size, unsigned dim, EMmeDataType type)
{
    for (unsigned i = 0; i < MAX_DIMENSION; ++i)
        if (size[i] == 0) size[i] = 1;
    return {size, (int) dim, type};
}
template<typename T>
static void fill(T val, unsigned n, MmeSimTensor& tensor, unsigned expBias = 0)
{
    DataBuffer data(n * sizeof(T));
    for (unsigned i = 0; i < n; i++) std::memcpy((T*) data + i, &val, sizeof(T));
    tensor.setData(data);
    if (tensor.getElementType() == e_type_fp8_152 || tensor.getElementType() == e_type_fp8_143) tensor.setFpBias(expBias);
}

static void gemm_simple_fp32()
{
    MmeSimTensor a = createSimTensor({5, 1}, 2, e_type_fp32), b = createSimTensor({1, 5}, 2, e_type_fp32);
    MmeSimTensor y = createSimTensor({1, 1}, 2, e_type_fp32);
    fill(10.0f, 5, a);
    fill(10.0f, 5, b);
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doBatchGemm(y, a, b, e_mme_ab);
    EXPECT(y.data() != nullptr);
    EXPECT(*(float*) y.data() == 500.0f);
}

static void gemm_api_simple_fp32()
{
    Matrix a(e_type_fp32, 1, 5), b(e_type_fp32, 5, 1), y(e_type_fp32, 1, 1);
    float val = 10.0f;
    DataBuffer data(5 * sizeof(float));
    for (unsigned i = 0; i < 5; i++) std::memcpy((float*) data + i, &val, sizeof(float));
    a.getMatrix().data = data;
    b.getMatrix().data = data;
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doGemm(y, a, b, false, false);
    EXPECT(*(float*) y.getMatrix().data.get() == 500.0f);
}

static void gemm_simple_bf16()
{
    MmeSimTensor a = createSimTensor({5, 1}, 2, e_type_bf16), b = createSimTensor({1, 5}, 2, e_type_bf16);
    MmeSimTensor y = createSimTensor({1, 1}, 2, e_type_fp32);
    bf16_t val(10, RoundingMode::RoundToNearest);
    fill(val, 5, a);
    fill(val, 5, b);
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doBatchGemm(y, a, b, e_mme_ab);
    EXPECT(*(float*) y.data() == 500.0f);
}

static void gemm_2d_fp32_ieee()
{
    MmeSimTensor a = createSimTensor({5, 5}, 2, e_type_fp32_ieee), b = createSimTensor({5, 5}, 2, e_type_fp32_ieee);
    MmeSimTensor y = createSimTensor({5, 5}, 2, e_type_fp32);
    fill(10.0f, 25, a);
    fill(5.0f, 25, b);
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doBatchGemm(y, a, b, e_mme_ab);
    for (unsigned i = 0; i < 25; i++) EXPECT(*((float*) y.data() + i) == 250.0f);
}

static void gemm_2d_bf16_with_activation()
{
    MmeSimTensor a = createSimTensor({5, 5}, 2, e_type_bf16), b = createSimTensor({5, 5}, 2, e_type_bf16);
    MmeSimTensor acc = createSimTensor({5, 5}, 2, e_type_fp32), y = createSimTensor({5, 5}, 2, e_type_bf16);
    bf16_t valA(10.0f), valB(5.0f);
    fill(valA, 25, a);
    fill(valB, 25, b);
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doBatchGemm(acc, a, b, e_mme_ab);
    pMMESimTensor pY = std::make_shared<MmeSimTensor>(y), pAcc = std::make_shared<MmeSimTensor>(acc);
    calculator.doActivation(pY, pAcc, nullptr, nullptr, false);
    for (unsigned i = 0; i < 25; i++)
    {
        bf16_t res(*(reinterpret_cast<uint16_t*>(pY->data()) + i));
        EXPECT((float) res == 250.0f);
    }
}

template<typename F8>
static void gemm_simple_fp8(EMmeDataType type, unsigned bias, float va, float vb)
{
    F8 valA(va, RoundingMode::RoundToNearest, bias), valB(vb, RoundingMode::RoundToNearest, bias);
    const float expected = valA.toFloat(bias) * valB.toFloat(bias) * 2;
    MmeSimTensor a = createSimTensor({2, 1}, 2, type), b = createSimTensor({1, 2}, 2, type);
    MmeSimTensor y = createSimTensor({1, 1}, 2, e_type_fp32);
    fill(valA, 2, a, bias);
    fill(valB, 2, b, bias);
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doBatchGemm(y, a, b, e_mme_ab);
    EXPECT(*(float*) y.data() == expected);
}

template<typename F8>
static void conv_fwd_fp8(EMmeDataType type, unsigned bias)
{
    MmeSimTensor a = createSimTensor({5, 5}, 2, type), w = createSimTensor({5, 5}, 2, type);
    MmeSimTensor y = createSimTensor({5, 5}, 2, e_type_fp32);
    fill((uint8_t) F8(0.5f, RoundingMode::RoundToNearest, bias), 25, a, bias);
    fill((uint8_t) F8(-0.5f, RoundingMode::RoundToNearest, bias), 25, w, bias);
    ConvolutionParams params;
    params.dim = 2;
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doConvolution(y, a, w, y, params, e_mme_fwd, RoundingMode::RoundToNearest);
    EXPECT(y.data() != nullptr);
    // x = [C=5, W=5], w = [K=5, C=5], 1x1 filter: every output is 5 * (0.5 * -0.5)
    for (unsigned i = 0; i < 25; i++) EXPECT(*((float*) y.data() + i) == -1.25f);
}

static void gemm_api_bf16_transposed()
{
    // mme_unit_test.cpp:539-575 uses fp16 operands, which this backend does not take; same shapes with bf16
    const unsigned M = 128, K = 128, N = 256;
    bf16_t val(10, RoundingMode::RoundToNearest);
    DataBuffer da(K * M * sizeof(uint16_t)), db(K * N * sizeof(uint16_t));
    for (unsigned i = 0; i < K * M; i++) std::memcpy((uint16_t*) da + i, &val, sizeof(uint16_t));
    for (unsigned i = 0; i < K * N; i++) std::memcpy((uint16_t*) db + i, &val, sizeof(uint16_t));
    Matrix a(e_type_bf16, K, M, da.get()), b(e_type_bf16, K, N, db.get()), y(e_type_fp32, M, N);
    CPUCalculator calculator(e_mme_Gaudi2);
    calculator.doGemm(y, a, b, true, false);
    for (unsigned i = 0; i < M * N; i += 97) EXPECT(*((float*) y.data() + i) == 100.0f * K);
}

static void unsupported_type_asserts()
{
    MmeSimTensor a = createSimTensor({5, 1}, 2, e_type_fp16), b = createSimTensor({1, 5}, 2, e_type_fp16);
    MmeSimTensor y = createSimTensor({1, 1}, 2, e_type_fp32);
    fill((uint16_t) 0x3c00, 5, a);
    fill((uint16_t) 0x3c00, 5, b);
    CPUCalculator calculator(e_mme_Gaudi3);
    bool threw = false;
    try
    {
        calculator.doBatchGemm(y, a, b, e_mme_ab);
    }
    catch (...)
    {
        threw = true;
    }
    EXPECT(threw);  // MME_ASSERT -> MMEStackException, never a silent CPU result
}

// fill_and_compare_float / fill_and_compare_bfloat16 / comparison_failure_bf16 (mme_unit_test.cpp:238-392) with the drop-in
// TensorComparator: the reference's generator and typed arithmetic build the tensors, the comparison runs on the GPU.
static void fill_and_compare()
{
    SizeArray sizes = {64, 32, 32, 64, 1};
    RandomSimTensorGenerator generator(1);
    {
        pMMESimTensor filled = std::make_shared<MmeSimTensor>(sizes, 4, e_type_fp32), acc = std::make_shared<MmeSimTensor>(sizes, 4, e_type_fp32);
        generator.fill(filled, 1035);
        float v = 0;
        for (unsigned count = 1; count < 46; count++) v += (float) count;
        for (unsigned e = 0; e < acc->getSizeInElements(); e++) ((float*) acc->data())[e] = v;
        TensorComparator comparator(false, e_type_fp32);
        EXPECT(comparator.doCompare(filled, "fillTensor", acc, "accumulatedTensor"));
        EXPECT(comparator.doCompareBitExact(filled, "fillTensor", acc, "accumulatedTensor"));
        EXPECT(!comparator.getDiffElement().is_set());
    }
    {
        pMMESimTensor filled = std::make_shared<MmeSimTensor>(sizes, 4, e_type_bf16), acc = std::make_shared<MmeSimTensor>(sizes, 4, e_type_bf16);
        generator.fill(filled, 1035);
        bf16_t v(0.0f);
        for (unsigned count = 1; count < 46; count++) v = bfloat16::add(v, bf16_t((float) count));
        for (unsigned e = 0; e < acc->getSizeInElements(); e++) ((bf16_t*) acc->data())[e] = v;
        TensorComparator comparator(false, e_type_bf16);
        EXPECT(comparator.doCompare(filled, "fillTensor", acc, "accumulatedTensor"));
        // from element 1000 on the values are 100 higher: reported, with the first difference at offset 1000
        const bf16_t bumped = bfloat16::add(v, bf16_t(100.0f));
        for (unsigned e = 1000; e < acc->getSizeInElements(); e++) ((bf16_t*) acc->data())[e] = bumped;
        EXPECT(!comparator.doCompare(filled, "fillTensor", acc, "accumulatedTensor", 0, "", 1, false));
        Settable<SizeArray> d = comparator.getDiffElement();
        EXPECT(d.is_set());
        if (d.is_set())
        {
            EXPECT(d.value()[0] + d.value()[1] * sizes[0] == 1000);
            EXPECT(d.value()[2] == 0 && d.value()[3] == 0 && d.value()[4] == 0);
        }
    }
    {
        Matrix a(e_type_fp32, 3, 4), b(e_type_fp32, 3, 4);
        for (unsigned e = 0; e < 12; e++) { ((float*) a.data())[e] = float(e); ((float*) b.data())[e] = float(e); }
        TensorComparator comparator(16, e_type_fp32);
        EXPECT(comparator.doCompare(a, "a", b, "b"));
        ((float*) b.data())[7] = 1000.0f;
        EXPECT(!comparator.doCompareBitExact(a, "a", b, "b"));
        EXPECT(comparator.getDiffElement().is_set() && comparator.getDiffElement().value()[0] == 1 && comparator.getDiffElement().value()[1] == 3);
    }
}

// transposed_dedx (mme_reference_impl.cpp:625-647): weights arrive as [C, K, S, R]; the calculator swaps the two fastest
// dims, mirrors S and runs dedx, whose col2im writes IN PLACE. Checked: the result lands in a caller-owned buffer that the
// output tensor does not own, and equals dedx on weights prepared by hand the same way.
static void transposed_dedx_in_place()
{
    const unsigned C = 8, K = 16, W = 6, H = 5, B = 2, S = 3, R = 3;
    SizeArray xs = {C, W, H, B, 1}, ws = {K, C, S, R, 1}, wts = {C, K, S, R, 1}, ys = {K, W, H, B, 1};
    const unsigned nx = C * W * H * B, nw = K * C * S * R, ny = K * W * H * B;
    MmeSimTensor w(ws, 4, e_type_bf16), wt(wts, 4, e_type_bf16), y(ys, 4, e_type_bf16);
    std::vector<uint16_t> wv(nw), wtv(nw), yv(ny);
    unsigned seed = 12345;
    auto next = [&]() { seed = seed * 1664525u + 1013904223u; return float(int((seed >> 20) & 15) - 8) * 0.25f; };
    for (auto& v : yv) v = (uint16_t) bf16_t(next(), RoundingMode::RoundToNearest);
    // w[k, c, s, r] (K fastest) drawn at random; wt[c, k, s', r] = w[k, c, S-1-s', r]
    for (unsigned i = 0; i < nw; i++) wv[i] = (uint16_t) bf16_t(next(), RoundingMode::RoundToNearest);
    for (unsigned r = 0; r < R; r++)
        for (unsigned s = 0; s < S; s++)
            for (unsigned c = 0; c < C; c++)
                for (unsigned k = 0; k < K; k++)
                    wtv[((r * S + (S - 1 - s)) * K + k) * C + c] = wv[((r * S + s) * C + c) * K + k];
    std::memcpy(w.data(), wv.data(), nw * 2);
    std::memcpy(wt.data(), wtv.data(), nw * 2);
    std::memcpy(y.data(), yv.data(), ny * 2);
    ConvolutionParams params;
    params.dim = 2;
    params.padding[0] = params.padding[1] = 1;
    CPUCalculator calculator(e_mme_Gaudi3);
    MmeSimTensor dx(xs, 4, e_type_fp32);
    calculator.doConvolution(dx, dx, w, y, params, e_mme_dedx, RoundingMode::RoundToNearest);
    // the caller's buffer, handed over without ownership and pre-filled with a marker
    std::vector<float> mine(nx, -77.0f);
    MmeSimTensor dxt(xs, 4, e_type_fp32, (char*) mine.data());
    EXPECT(dxt.data() == (char*) mine.data());
    calculator.doConvolution(dxt, dxt, wt, y, params, e_mme_transposed_dedx, RoundingMode::RoundToNearest);
    EXPECT(dxt.data() == (char*) mine.data());   // still the caller's buffer: no fresh allocation was swapped in
    unsigned diff = 0, nonzero = 0;
    for (unsigned i = 0; i < nx; i++)
    {
        diff += mine[i] != ((float*) dx.data())[i];
        nonzero += mine[i] != 0.0f;
    }
    EXPECT(diff == 0);
    EXPECT(nonzero > nx / 2);
}

int main()
{
    gemm_simple_fp32();
    gemm_api_simple_fp32();
    gemm_simple_bf16();
    gemm_2d_fp32_ieee();
    gemm_2d_bf16_with_activation();
    gemm_simple_fp8<fp8_143_t>(e_type_fp8_143, 7, 0.25f, -0.5f);
    gemm_simple_fp8<fp8_152_t>(e_type_fp8_152, EXPONENT_BIAS_FP8_152_15, 0.5f, -0.5f);
    conv_fwd_fp8<fp8_143_t>(e_type_fp8_143, 3);
    conv_fwd_fp8<fp8_152_t>(e_type_fp8_152, EXPONENT_BIAS_FP8_152_15);
    gemm_api_bf16_transposed();
    unsupported_type_asserts();
    fill_and_compare();
    transposed_dedx_in_place();
    std::printf(g_failures ? "shim unit tests: %d FAILED\n" : "shim unit tests: all passed\n", g_failures);
    return g_failures ? 1 : 0;
}
