// Synapse-facing calculator helpers on the B200 backend.
//
// Same names, arguments and meaning as the helpers of synapse/tests/utils/cpu_calculator.h:20-249, so a
// Synapse test links this translation unit in place of synapse/tests/utils/cpu_calculator.cpp. The
// difference is where the work happens: operands are uploaded once, convolution / GEMM, the rounded cast
// and the comparison all run on the GPU through the C ABI (include/mme_b200.h), and the check* functions
// bring back only the verdict, the first differing coordinate and the expected value there.
//
// Built against the Synapse public header (synapse/include/synapse_common_types.h: synTensorDescriptor,
// synConvolution3DParams, synGEMMParams, synDeviceType, synDataType) and mme_common_enum.h (RoundingMode).
#pragma once

#include <array>

#include "include/mme_common/mme_common_enum.h"
#include "synapse_common_types.h"

// graph_compiler/types.h:107 defines the same alias; repeating an identical alias is legal C++.
using CoordArray = std::array<int, SYN_MAX_TENSOR_DIM>;

// The misspelling is the reference's (cpu_calculator.h:7-17); kept so callers compile unchanged.
typedef enum
{
    REFERENCE_OP_FWD,
    REFERENCE_OP_DEDX,
    REFERENCE_OP_DEDW,
    REFERENCE_OP_AB,
    REFERENCE_OP_ABT,
    REFERENCE_OP_ATB,
    REFERENCE_OP_ATBT,
    REFERENCE_OP_TRANSPOSED_DEDX,
} ERepefenceOp;

// Value of the element at wrongIdx, as float (cpu_calculator.cpp:115-125: bf16 buffers return the raw
// 16-bit pattern converted to float, everything else is read as float).
float getIndexValue(const TSize* sizes, const CoordArray& wrongIdx, synDataType type, void* buffer);

// |a-b| <= abstol + reltol*min(|a|,|b|) per element with the tolerances of cpu_calculator.cpp:211-223
// (bf16: 1e-6 / 0.015, else 1e-7 / 0.0015); NaN equals NaN. Runs on the host: it is a two-buffer scan
// with no arithmetic worth a launch.
bool checkResults(const synTensorDescriptor& desc, char* firstData, char* secondData, CoordArray& outIndex);

// cpu_calculator.cpp:383-486. usePearsonComparison replaces the element-wise comparator by the statistical rule of the
// device tests (synapse/tests/utils/tensor_validator.inl:171-187: Pearson correlation >= 0.95 and an L2-norm ratio >= 0.8
// for results longer than 15 elements); the reference raises gtest failures from inside that helper, here the verdict is
// the return value. bf16 and fp32 results only.
bool checkMmeOp(const synTensorDescriptor& xDesc, char* xData, const synTensorDescriptor& wDesc, char* wData,
                const synTensorDescriptor& yDesc, char* yData, const synConvolution3DParams& convParams, ERepefenceOp op,
                CoordArray& outIndex, synDeviceType deviceType, float* expectedResult = nullptr,
                bool usePearsonComparison = false,
                MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);

// cpu_calculator.cpp:488-585.
bool checkBatchGemmOp(const synTensorDescriptor& xDesc, char* xData, const synTensorDescriptor& wDesc, char* wData,
                      const synTensorDescriptor& yDesc, char* yData, ERepefenceOp op, CoordArray& outIndex,
                      float* expectedResult, synDeviceType deviceType,
                      MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);

// cpu_calculator.cpp:587-668: y = cast(x.w + xMask.wMask), both products accumulated in fp32 and added in fp32.
bool checkMaskedBatchGemmOp(const synTensorDescriptor& xDesc, char* xData, const synTensorDescriptor& wDesc, char* wData,
                            const synTensorDescriptor& xMaskDesc, char* xMaskData, const synTensorDescriptor& wMaskDesc,
                            char* wMaskData, const synTensorDescriptor& yDesc, char* yData, ERepefenceOp op,
                            CoordArray& outIndex, float* expectedResult, synDeviceType deviceType,
                            MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);

// cpu_calculator.cpp:677-750.
bool checkFwdConvolution(const synTensorDescriptor& x, char* xData, const synTensorDescriptor& w, char* wData,
                         const synTensorDescriptor& y, char* yData, const synConvolution3DParams& convParams,
                         CoordArray& outIndex, synDeviceType deviceType,
                         MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);
bool checkDEDX(const synTensorDescriptor& y, char* yData, const synTensorDescriptor& w, char* wData,
               const synTensorDescriptor& x, char* xData, const synConvolution3DParams& convParams, CoordArray& outIndex,
               synDeviceType deviceType, MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);
bool checkDEDW(const synTensorDescriptor& y, char* yData, const synTensorDescriptor& x, char* xData,
               const synTensorDescriptor& w, char* wData, const synConvolution3DParams& convParams, CoordArray& outIndex,
               synDeviceType deviceType, bool usePearsonCompare = false,
               MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);

// cpu_calculator.cpp:752-790: result = cast(conv(...)) in the output descriptor's dtype, ReLU from convParams.
void calculateFwdConvolution(const synTensorDescriptor& x, char* xData, const synTensorDescriptor& w, char* wData,
                             const synTensorDescriptor& y, char* result, const synConvolution3DParams& convParams,
                             synDeviceType deviceType,
                             MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);
void calculateDEDX(const synTensorDescriptor& y, char* yData, const synTensorDescriptor& w, char* wData,
                   const synTensorDescriptor& x, char* result, const synConvolution3DParams& convParams,
                   synDeviceType deviceType, MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);
void calculateDEDW(const synTensorDescriptor& y, char* yData, const synTensorDescriptor& x, char* xData,
                   const synTensorDescriptor& w, char* result, const synConvolution3DParams& convParams,
                   synDeviceType deviceType, MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);

// cpu_calculator.cpp:823-834 (params.transpose_* are ignored there too: `op` carries the orientation).
void calculateGemm(const synTensorDescriptor& xDesc, char* xData, const synTensorDescriptor& wDesc, char* wData,
                   const synTensorDescriptor& yDesc, char* yData, const synGEMMParams& params, ERepefenceOp op,
                   synDeviceType deviceType, MmeCommon::RoundingMode roundingMode = MmeCommon::RoundingMode::RoundToNearest);

// cpu_calculator.cpp:849-863: out = float(a) + float(b) in the descriptor's type (fp32 on the GPU; bf16 on the host).
void calculateAdd(const synTensorDescriptor& desc, char* inA, char* inB, char* out);
