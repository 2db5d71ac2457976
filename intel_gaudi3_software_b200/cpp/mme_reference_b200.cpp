// Drop-in replacement for the reference's calculator implementation
// (mme/mme_reference/mme_reference_impl.cpp): this translation unit defines every member of Matrix
// and CPUCalculator that the reference's public header (mme/mme_reference/mme_reference.h:60-191)
// declares, and forwards the calculator's work to the B200 backend through the C ABI
// (include/mme_b200.h). It is compiled against the reference's own headers and linked with the
// reference's sim_tensor*.cpp in place of mme_reference_impl.cpp; callers do not change.
//
// Semantics kept from the reference:
//   - doBatchGemm, dedx and transposed_dedx write into the output tensor's buffer in place, through its
//     strides (col2im, mme_reference_impl.cpp:858-861); fwd / dedw / the doDma transposes give the output
//     tensor a fresh buffer (mme_reference_impl.cpp:862-868, 396-428);
//   - failures surface as MME_ASSERT (mme/include/mme_assert.h:27-60);
//   - one calculator = one host thread at a time.
// Not available on this backend (asserts): integer / gemmlowp paths (zeroPoints, ActivationParams),
// fp16 / ufp16 operands.
#include <cstring>
#include <string>

#include "mme_reference.h"
#include "include/mme_assert.h"
#include "mme_b200.h"

using namespace MmeCommon;

// ------------------------------------------------------------------------------------------ Matrix
static unsigned elementBytes(EMmeDataType type)
{
    switch (type)
    {
        case e_type_fp8_143:
        case e_type_fp8_152:
        case e_type_int8:
        case e_type_uint8:
        case e_type_int4:
        case e_type_uint4:
            return 1;
        case e_type_bf16:
        case e_type_fp16:
        case e_type_ufp16:
        case e_type_int16:
        case e_type_uint16:
            return 2;
        case e_type_fp32:
        case e_type_fp32_ieee:
        case e_type_tf32:
        case e_type_int32:
        case e_type_int32_26:
        case e_type_int32_16:
            return 4;
        default:
            MME_ASSERT(0, "type not supported");
    }
    return 0;
}

Matrix::Matrix(EMmeDataType type, uint64_t height, uint64_t width, byte* data, const bool shouldCopyData)
: m_type(type), m_matrixDataPtr(nullptr)
{
    setInternalMatrixSizes(type, height, width);
    const uint64_t bytes = height * width * m_matrix.sizeOfDataType;
    m_matrix.data = data ? DataBuffer(data, bytes, shouldCopyData) : DataBuffer(bytes);
}

Matrix::Matrix(EMmeDataType type, uint64_t height, uint64_t width, uint64_t inputElementStride, const byte* inputDataPtr)
: m_type(type)
{
    // gathers `height` rows of `width` elements that lie (width + inputElementStride) elements apart
    setInternalMatrixSizes(type, height, width);
    const uint64_t es = m_matrix.sizeOfDataType;
    m_matrixDataPtr = new byte[height * width * es];
    for (uint64_t r = 0; r < height; ++r)
        std::memcpy(m_matrixDataPtr + r * width * es, inputDataPtr + r * (width + inputElementStride) * es, width * es);
    m_matrix.data = DataBuffer(m_matrixDataPtr, height * width * es, false);
}

Matrix::~Matrix()
{
    delete[] m_matrixDataPtr;
}

void Matrix::setInternalMatrixSizes(EMmeDataType type, uint64_t height, uint64_t width)
{
    m_matrix.setShape(height, width);
    m_matrix.sizeOfDataType = elementBytes(type);
}

void Matrix::doTranspose()
{
    getMatrix().doTranspose();
}

void Matrix::getDataWithStride(uint64_t height, uint64_t width, byte* outputDataPtr, int outputElementSize, uint64_t outputStride)
{
    for (uint64_t r = 0; r < height; ++r)
        std::memcpy(outputDataPtr + r * (width + outputStride) * outputElementSize,
                    m_matrix.data.get() + r * width * outputElementSize, width * outputElementSize);
}

// ------------------------------------------------------------------------------------------ implementation object
class CPUCalculatorImpl
{
public:
    CPUCalculatorImpl(ChipType chip, unsigned seed, uint32_t lfsrNumRegs, uint32_t* lfsr, uint32_t polynomial)
    {
        int device = 0;
        if (const char* env = std::getenv("MME_B200_DEVICE")) device = std::atoi(env);
        const int rc = mmeb200_create(&ctx, (int) chip, device, seed, lfsrNumRegs, lfsr, polynomial);
        MME_ASSERT(rc == 0, rc == MMEB200_ERR_NO_DEVICE ? "mme_b200: no B200 visible (there is no CPU fallback)"
                                                        : "mme_b200: could not create the backend context");
        // MME_B200_ACCUMULATION=exact: the reference's Gaudi3 arithmetic on the GPU (bit-identical accumulators) instead
        // of the tensor cores; the constructor's signature stays the reference's, so the choice comes from the environment.
        if (const char* env = std::getenv("MME_B200_ACCUMULATION"))
            if (std::string(env) == "exact" && chip == e_mme_Gaudi3) check(mmeb200_set_accumulation(ctx, MMEB200_ACC_CHIP_EXACT));
    }
    ~CPUCalculatorImpl() { mmeb200_destroy(ctx); }
    void check(int rc) const
    {
        if (rc != 0)
        {
            const std::string msg = std::string("mme_b200: ") + mmeb200_last_error(ctx);
            MME_ASSERT(rc == 0, msg.c_str());
        }
    }
    mmeb200_ctx* ctx = nullptr;
};

static mmeb200_tensor describe(const MMESimTensorBase& t, void* data)
{
    mmeb200_tensor d;
    std::memset(&d, 0, sizeof d);
    d.dtype = (int) t.getElementType();
    d.dims = t.getDim();
    for (int i = 0; i < MMEB200_MAX_DIMS; i++)
    {
        d.sizes[i] = (uint32_t) t.getSize(i);
        d.strides[i] = (uint32_t) t.getStride(i);
    }
    d.fp_bias = t.getFpBias();
    d.inf_nan_mode = (int) t.getInfNanMode();
    d.mem_space = MMEB200_MEM_HOST;
    d.data = data;
    return d;
}

static mmeb200_tensor describe(const Matrix& m, unsigned fpBias, InfNanMode mode)
{
    mmeb200_tensor d;
    std::memset(&d, 0, sizeof d);
    d.dtype = (int) m.getElementType();
    d.dims = 2;
    d.sizes[0] = (uint32_t) m.getMatrix().getWidth();
    d.sizes[1] = (uint32_t) m.getMatrix().getHeight();
    d.strides[0] = 1;
    d.strides[1] = d.sizes[0];
    for (int i = 2; i < MMEB200_MAX_DIMS; i++)
    {
        d.sizes[i] = 1;
        d.strides[i] = d.sizes[0] * d.sizes[1];
    }
    d.fp_bias = fpBias;
    d.inf_nan_mode = (int) mode;
    d.mem_space = MMEB200_MEM_HOST;
    d.data = const_cast<byte*>(m.data());
    return d;
}

// ------------------------------------------------------------------------------------------ CPUCalculator
CPUCalculator::CPUCalculator(ChipType chip, int max_tensor_dims, int max_conv_dims, unsigned seed, uint32_t lfsrNumRegs,
                             uint32_t* lfsr, uint32_t polynomial)
{
    MME_ASSERT(max_tensor_dims == MME_MAX_TENSOR_DIMS, "dynamic value different than static value");
    MME_ASSERT(max_conv_dims == MME_MAX_CONV_DIMS, "dynamic value different than static value");
    m_impl = std::make_unique<CPUCalculatorImpl>(chip, seed, lfsrNumRegs, lfsr, polynomial);
}

CPUCalculator::~CPUCalculator() = default;

void CPUCalculator::limitNumOfThreads(unsigned numOfThreads)
{
    m_impl->check(mmeb200_limit_num_of_threads(m_impl->ctx, numOfThreads));
}

void CPUCalculator::doGemm(Matrix& output, const Matrix& inputA, const Matrix& inputB, bool transposeA, bool transposeB,
                           RoundingMode rm, unsigned fpBiasA, unsigned fpBiasB, bool clipFp, bool clipFpInfIn,
                           InfNanMode infNanModeA, InfNanMode infNanModeB, int* zeroPoints)
{
    MME_ASSERT(zeroPoints == nullptr, "mme_b200: integer paths are not supported");
    mmeb200_tensor o = describe(output, 0, e_mme_full_inf_nan);
    mmeb200_tensor a = describe(inputA, fpBiasA, infNanModeA), b = describe(inputB, fpBiasB, infNanModeB);
    const int op = transposeA ? (transposeB ? MMEB200_OP_ATBT : MMEB200_OP_ATB) : (transposeB ? MMEB200_OP_ABT : MMEB200_OP_AB);
    m_impl->check(mmeb200_bgemm(m_impl->ctx, &o, &a, &b, op, nullptr));
}

void CPUCalculator::doDma(MmeSimTensor& outputTensor, const MmeSimTensor& xTensor, EMmeOpType op)
{
    switch (op)
    {
        case e_mme_memcpy:
            outputTensor = xTensor;
            return;
        case e_mme_gemm_transpose:
        case e_mme_trans:
        {
            DataBuffer fresh(outputTensor.getMemorySize());
            mmeb200_tensor o = describe(outputTensor, fresh.get()), x = describe(xTensor, xTensor.data());
            m_impl->check(mmeb200_dma(m_impl->ctx, &o, &x, MMEB200_OP_TRANS));
            outputTensor.setData(fresh);
            return;
        }
        default:
            MME_ASSERT(0, "invalid dma op");
    }
}

void CPUCalculator::doBatchGemm(MmeSimTensor& outputTensor, const MmeSimTensor& xTensor, const MmeSimTensor& wTensor,
                                EMmeOpType op, RoundingMode rm, bool clipFp, bool clipFpInfIn, int* zeroPoints)
{
    MME_ASSERT(zeroPoints == nullptr, "mme_b200: integer paths are not supported");
    mmeb200_tensor o = describe(outputTensor, outputTensor.data());
    mmeb200_tensor x = describe(xTensor, xTensor.data()), w = describe(wTensor, wTensor.data());
    m_impl->check(mmeb200_bgemm(m_impl->ctx, &o, &x, &w, (int) op, nullptr));
}

void CPUCalculator::doConvolution(MmeSimTensor& outputTensor, const MmeSimTensor& xTensor, const MmeSimTensor& wTensor,
                                  const MmeSimTensor& yTensor, const ConvolutionParams& params, EMmeOpType op,
                                  RoundingMode rm, bool clipFp, bool clipFpInfIn, int* zeroPoints)
{
    MME_ASSERT(zeroPoints == nullptr, "mme_b200: integer paths are not supported");
    mmeb200_conv_params p;
    std::memset(&p, 0, sizeof p);
    p.dim = params.dim;
    for (int i = 0; i < MMEB200_MAX_CONV_DIMS; i++)
    {
        p.padding[i] = params.padding[i];
        p.stride[i] = params.convStride[i];
        p.dilation[i] = params.dilation[i];
    }
    p.padding_value = params.paddingValue.int32;
    p.relu = params.relu;
    mmeb200_tensor x = describe(xTensor, xTensor.data()), w = describe(wTensor, wTensor.data()), y = describe(yTensor, yTensor.data());
    if (op == e_mme_dedx || op == e_mme_transposed_dedx)
    {
        // both end in RefIm2Col::doCol2Im, which writes in place through the tensor's strides: a caller-owned
        // (non-owning) buffer receives the result and the gaps of a strided tensor keep their contents
        mmeb200_tensor o = describe(outputTensor, outputTensor.data());
        m_impl->check(mmeb200_conv(m_impl->ctx, &o, &x, &w, &y, &p, (int) op, (int) rm, nullptr));
        return;
    }
    // fwd / dedw: the reference hands the output tensor a newly built buffer
    DataBuffer fresh(outputTensor.getMemorySize());
    mmeb200_tensor o = describe(outputTensor, fresh.get());
    m_impl->check(mmeb200_conv(m_impl->ctx, &o, &x, &w, &y, &p, (int) op, (int) rm, nullptr));
    outputTensor.setData(fresh);
}

void CPUCalculator::doActivation(pMMESimTensor output, const pMMESimTensor acc, const pMMESimTensor res, const pMMESimTensor bias,
                                 bool relu, RoundingMode rm, const ActivationParams* actParams, bool clipFp, bool clipInfIn,
                                 bool flushDenorms, bool stochasticFTZfp8)
{
    MME_ASSERT(actParams == nullptr, "mme_b200: the gemmlowp activation path is not supported");
    mmeb200_cast_params c;
    std::memset(&c, 0, sizeof c);
    c.rounding = (int) rm;
    c.relu = relu;
    c.clip_fp = clipFp;
    c.clip_inf_in = clipInfIn;
    c.flush_denorms = flushDenorms;
    c.stochastic_ftz_fp8 = stochasticFTZfp8;
    c.rng_kind = MMEB200_RNG_LFSR;  // the calculator's own LFSR registers, advanced like m_lfsr
    mmeb200_tensor o = describe(*output, output->data()), a = describe(*acc, acc->data());
    m_impl->check(mmeb200_activation(m_impl->ctx, &o, &a, &c));
}

void CPUCalculator::doMemoryWrite(pMMESimTensor memory, const pMMESimTensor mmeOut, EMmeReductionOp reductionOp,
                                  EMmeReductionRm reductionRm, bool clipFp)
{
    mmeb200_tensor m = describe(*memory, memory->data()), o = describe(*mmeOut, mmeOut->data());
    m_impl->check(mmeb200_memory_write(m_impl->ctx, &m, &o, (int) reductionOp, (int) reductionRm, clipFp));
}

void CPUCalculator::activationGemmlowp(pMMESimTensor, pMMESimTensor, pMMESimTensor, pMMESimTensor, bool, RoundingMode,
                                       const ActivationParams*)
{
    MME_ASSERT(0, "mme_b200: the gemmlowp activation path is not supported");
}
