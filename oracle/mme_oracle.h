/*
 * TEST INFRASTRUCTURE -- CPU restatement of the Gaudi MME compute reference ("the oracle port").
 *
 * Only tests/, the smoke check and the CPU-baseline leg of the benchmark may load this. It is
 * never linked into, imported by or called from the product library.
 *
 * Parity status: PINNED. Every function here is checked (tests/test_oracle_*.py) against the
 * reference's own known-answer unit tests (mme/tests/unit_tests/mme_unit_test.cpp) and against
 * golden vectors produced by running the compiled, unmodified reference (oracle/_ref) -- see
 * tests/golden/make_golden.py.
 *
 * Scope of the restatement: the Gaudi3 chip model for bf16 and fp8 operands (the formats of the
 * hot path), all conversions, activation, im2col / col2im lowering and memory-write add. The
 * fp32 / tf32 operand models and the Gaudi / Gaudi2 chip models are exercised through oracle/_ref.
 */
#ifndef MME_ORACLE_H
#define MME_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* same plain-data layout as mmeb200_tensor / mmeb200_conv_params / mmeb200_cast_params */
typedef struct {
    int32_t dtype, dims;
    uint32_t sizes[5], strides[5];
    uint32_t fp_bias;
    int32_t inf_nan_mode, mem_space, reserved;
    void* data;
} mo_tensor;
typedef struct {
    int32_t dim, padding[4], stride[4], dilation[4];
    uint32_t padding_value;
    int32_t relu;
} mo_conv_params;
typedef struct {
    int32_t rounding, relu, clip_fp, clip_inf_in, flush_denorms, stochastic_ftz_fp8, rng_kind, reserved;
    uint64_t rng_seed, rng_offset;
} mo_cast_params;

/* scalar conversions */
uint32_t mo_fp8_to_fp32(uint8_t v, int exp_width, unsigned bias, int inf_nan_mode);
uint8_t mo_fp32_to_fp8(uint32_t bits, int exp_width, unsigned bias, int rm, uint32_t lfsr, int ftz, int clip,
                       int clip_inf_in, int stochastic_ftz, int inf_nan_mode);
uint16_t mo_fp32_to_bf16(uint32_t bits, int rm, uint32_t lfsr, int clip, int ftz, int clip_inf_in);
uint32_t mo_fp32_to_fp32(uint32_t bits, int rm, int clip, int ftz, int clip_inf_in);
uint32_t mo_lfsr32(uint32_t v, uint32_t poly);
void mo_fp32_to_bf16_vec(const uint32_t* in, uint16_t* out, size_t n, int rm, const uint32_t* lfsr, int clip, int ftz,
                         int clip_inf_in);
void mo_fp32_to_fp8_vec(const uint32_t* in, uint8_t* out, size_t n, int exp_width, unsigned bias, int rm,
                        const uint32_t* lfsr, int ftz, int clip, int clip_inf_in, int stochastic_ftz, int mode);
void mo_fp8_to_fp32_vec(const uint8_t* in, uint32_t* out, size_t n, int exp_width, unsigned bias, int mode);

/* one Gaudi3 tree step: 8 products + accumulator, operands already decoded to fp32 bits */
uint32_t mo_tree8_acc(const uint32_t a[8], const uint32_t b[8], uint32_t c);
/* K-long dot product under the Gaudi3 model; dtype = EMmeDataType value (bf16, fp8_143, fp8_152) */
float mo_fma_vec(int type_a, int type_b, unsigned bias_a, unsigned bias_b, int mode_a, int mode_b, const void* a,
                 const void* b, unsigned n);

/* calculator-level operations (Gaudi3 model); return 0 on success */
int mo_bgemm(int threads, mo_tensor* out, const mo_tensor* x, const mo_tensor* w, int op);
int mo_conv(int threads, mo_tensor* out, const mo_tensor* x, const mo_tensor* w, const mo_tensor* y,
            const mo_conv_params* p, int op, int rm);
int mo_activation(mo_tensor* out, mo_tensor* acc, const mo_cast_params* c, uint32_t* lfsr, uint32_t num_regs,
                  uint32_t polynomial);
int mo_memory_write(mo_tensor* mem, const mo_tensor* mme_out, int op, int rm, int clip);
int mo_hardware_threads(void);

#ifdef __cplusplus
}
#endif
#endif
