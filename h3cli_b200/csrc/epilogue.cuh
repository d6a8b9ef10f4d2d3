/* The fused epilogue shared by every linear kernel in this library.
 *
 * It reproduces, in registers, the reference's unfused operator chain
 *   linear (+bias) -> bf16 | GELU-tanh (bf16 -> bf16) | gate*branch + residual (bf16 -> bf16)
 * including each intermediate bf16 rounding, so that "one fused kernel" and
 * "GEMM kernel followed by elementwise kernels" give the same bits for the same
 * accumulator.  The reference compiles with --fmad=false (Makefile:117), hence
 * the explicit __fmul_rn / __fadd_rn: no multiply-add contraction anywhere.
 *
 * Formulas followed:
 *   bias      src/metal/shaders.metal:855          bf16(acc + float(bias[n]))
 *   W8A8      src/metal/shaders.metal:2463-2464    bf16((float(acc) * in_scale[r]) * w_scale[n])
 *   GELU-tanh src/cuda/cuda_kernels.cuh:883-893
 *   gate      src/cuda/cuda_kernels.cuh:979-984    bf16(float(res) + float(branch) * float(gate[n]))
 */
#pragma once
#include "sm100_ptx.cuh"

namespace h3q8 {

enum : uint32_t { ACT_NONE = 0, ACT_GELU_TANH = 1 };

/* Device view of the optional epilogue operands (all may be null). */
struct EpilogueParams {
    const uint16_t *bias;      /* bf16 [N]   */
    const uint16_t *gate;      /* bf16 [N]   */
    const uint16_t *residual;  /* bf16 [M,N] */
    uint32_t activation;
};

__device__ __forceinline__ float gelu_tanh_f32(float v) {
    float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, cube));
    if (inner <= -10.0f) return 0.0f;
    if (inner >= 10.0f) return v;
    /* 0.5 v (1 + tanh u) == v / (1 + exp(-2u)).  The exponential and the division
     * use the hardware approximations (relative error about 1e-6), far inside the
     * bf16 rounding that follows; against a correctly rounded tanhf the stored
     * bf16 differs by one step for a few outputs in ten thousand. */
    return __fdividef(v, 1.0f + __expf(-2.0f * inner));
}

/* linear: fp32 linear result before bias.  Returns the final bf16 bits. */
__device__ __forceinline__ uint32_t epilogue_value(float linear, float bias, bool has_bias,
                                                   uint32_t activation, bool gated, float gate,
                                                   float residual) {
    if (has_bias) linear = __fadd_rn(linear, bias);
    uint32_t y = f32_to_bf16_bits(linear);
    if (activation == ACT_GELU_TANH) y = f32_to_bf16_bits(gelu_tanh_f32(bf16_bits_to_f32(y)));
    if (gated) y = f32_to_bf16_bits(__fadd_rn(residual, __fmul_rn(bf16_bits_to_f32(y), gate)));
    return y;
}

} /* namespace h3q8 */
