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

enum : uint32_t { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_SWIGLU = 2, ACT_QKV_ROPE = 3 };

/* QKV epilogue of the DiT block (src/cuda/cuda_kernels.cuh:988-1045, grouped layout
 * src/gpu.h:652-653): output columns are [head, q/k/v, 128]; q and k get a per-head RMS
 * norm with a learned weight and rotary embedding on the first 2*rope_half dimensions,
 * v is copied; all three are stored as [row, head, 128]. */
struct RopeParams {
    const uint16_t *q_norm, *k_norm;   /* bf16 [128]                 */
    const uint16_t *cos, *sin;         /* bf16 [rows, rope_half]     */
    uint16_t *query, *key, *value;     /* bf16 [rows, heads, 128]    */
    uint32_t heads, rope_half;         /* rope_half: 48 or 64        */
    float epsilon;
};

/* Device view of the optional epilogue operands (all may be null). */
struct EpilogueParams {
    const uint16_t *bias;      /* bf16 [N]   */
    const uint16_t *gate;      /* bf16 [N]   */
    const uint16_t *residual;  /* bf16 [M,N] */
    uint32_t activation;
    RopeParams rope;           /* used when activation == ACT_QKV_ROPE */
};

/* Branch-free so that the compiler can interleave many elements per thread.
 *   s = v + 0.044715 v^3,   0.5 v (1 + tanh(c s)) == v / (1 + exp(-2 c s)),   exp(-2 c s) = 2^(s * (-2 c log2 e))
 * The constants of the exponent are folded into one multiply; the exponential and the reciprocal are the hardware
 * approximations (relative error about 1e-6), far inside the bf16 rounding that follows; against a correctly rounded
 * tanhf the stored bf16 differs by one step for a few outputs in ten thousand.  The reference's lower saturation
 * guard (c s <= -10 -> 0) is kept as a select; its upper guard (c s >= 10 -> v) needs none: there 1 + exp(-2 c s)
 * rounds to 1 and v / 1 is v. */
__device__ __forceinline__ float gelu_tanh_f32(float v) {
    const float s = __fadd_rn(v, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v));
    float e, q;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(s, -2.3022082f)));   /* -2 sqrt(2/pi) log2(e) */
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q) : "f"(__fadd_rn(1.0f, e)));
    const float r = __fmul_rn(v, q);
    return s <= -12.533141f ? 0.0f : r;   /* c s <= -10 */
}

/* Round two fp32 values to bf16 (nearest even, one cvt.rn.bf16x2.f32) and keep them
 * packed: low half = first value.  Equal to the reference's bit recipe for every
 * finite input. */
__device__ __forceinline__ uint32_t pack_bf16_pair(float lo, float hi) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

/* Two adjacent outputs at once.  lin*: fp32 linear results before bias; bias, gate,
 * residual: packed bf16 pairs.  Returns the final packed bf16 pair. */
__device__ __forceinline__ uint32_t epilogue_pair(float lin0, float lin1, uint32_t bias, bool has_bias, uint32_t activation,
                                                  bool gated, uint32_t gate, uint32_t residual) {
    if (has_bias) { lin0 = __fadd_rn(lin0, bf16_lo(bias)); lin1 = __fadd_rn(lin1, bf16_hi(bias)); }
    uint32_t y = pack_bf16_pair(lin0, lin1);
    if (activation == ACT_GELU_TANH) y = pack_bf16_pair(gelu_tanh_f32(bf16_lo(y)), gelu_tanh_f32(bf16_hi(y)));
    if (gated) y = pack_bf16_pair(__fadd_rn(bf16_lo(residual), __fmul_rn(bf16_lo(y), bf16_lo(gate))),
                                  __fadd_rn(bf16_hi(residual), __fmul_rn(bf16_hi(y), bf16_hi(gate))));
    return y;
}

/* SwiGLU of the fc1 projection whose weight rows are [gate (N) | up (N)]:
 *   out = bf16( gate_b / (1 + exp(-gate_b)) * up ),  gate_b = bf16(gate linear result)
 * up stays fp32 on the int8 path (src/metal/shaders.metal:2269-2314) and is the bf16
 * linear output on the bf16 / W8A16 path, where the reference runs h3_swiglu_bf16 on the
 * stored [M, 2N] tensor (src/cuda/cuda_kernels.cuh:1047-1059). */
__device__ __forceinline__ float swiglu_f32(float gate_linear, float up_linear, bool round_up) {
    const float gate = bf16_lo(pack_bf16_pair(gate_linear, 0.0f));
    const float up = round_up ? bf16_lo(pack_bf16_pair(up_linear, 0.0f)) : up_linear;
    return __fmul_rn(__fdividef(gate, 1.0f + __expf(-gate)), up);
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

/* One (row, head, q-or-k) stream held by one thread: xp = its 128 linear outputs, already
 * rounded to bf16 and packed in pairs; sum = sum of their squares accumulated in dimension
 * order with fmaf, as the reference's loop does.  Writes the 128 normalised, rotated values. */
template <int ROPE_HALF>
__device__ __forceinline__ void qkv_rope_store(const uint32_t (&xp)[64], float sum, const uint16_t *__restrict__ norm_weight,
                                               const uint16_t *__restrict__ cos_row, const uint16_t *__restrict__ sin_row,
                                               float epsilon, uint16_t *__restrict__ dst) {
    static_assert(ROPE_HALF % 8 == 0 && 2 * ROPE_HALF <= 128, "rotary half must be a multiple of 8 within the head");
    const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(sum, 128.0f), epsilon));
    /* eight dimensions at a time; the rotary partner of a group of eight is another aligned group of eight */
#pragma unroll
    for (int g = 0; g < 16; g++) {
        const int d0 = g * 8;
        const bool rotary = d0 < 2 * ROPE_HALF, low = d0 < ROPE_HALF;
        const int p0 = low ? d0 + ROPE_HALF : d0 - ROPE_HALF;        /* partner group (unused when !rotary) */
        const int f0 = low ? d0 : d0 - ROPE_HALF;                     /* cos/sin index of the group          */
        uint32_t w[4], wp[4] = {0, 0, 0, 0}, c[4] = {0, 0, 0, 0}, sn[4] = {0, 0, 0, 0}, out[4];
        *reinterpret_cast<uint4 *>(w) = reinterpret_cast<const uint4 *>(norm_weight)[g];
        if (rotary) {
            *reinterpret_cast<uint4 *>(wp) = reinterpret_cast<const uint4 *>(norm_weight)[p0 / 8];
            *reinterpret_cast<uint4 *>(c) = reinterpret_cast<const uint4 *>(cos_row)[f0 / 8];
            *reinterpret_cast<uint4 *>(sn) = reinterpret_cast<const uint4 *>(sin_row)[f0 / 8];
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float v0 = __fmul_rn(__fmul_rn(bf16_lo(xp[d0 / 2 + j]), inverse), bf16_lo(w[j]));
            float v1 = __fmul_rn(__fmul_rn(bf16_hi(xp[d0 / 2 + j]), inverse), bf16_hi(w[j]));
            if (rotary) {
                const float o0 = __fmul_rn(__fmul_rn(bf16_lo(xp[p0 / 2 + j]), inverse), bf16_lo(wp[j]));
                const float o1 = __fmul_rn(__fmul_rn(bf16_hi(xp[p0 / 2 + j]), inverse), bf16_hi(wp[j]));
                if (low) {
                    v0 = __fsub_rn(__fmul_rn(v0, bf16_lo(c[j])), __fmul_rn(o0, bf16_lo(sn[j])));
                    v1 = __fsub_rn(__fmul_rn(v1, bf16_hi(c[j])), __fmul_rn(o1, bf16_hi(sn[j])));
                } else {
                    v0 = __fadd_rn(__fmul_rn(v0, bf16_lo(c[j])), __fmul_rn(o0, bf16_lo(sn[j])));
                    v1 = __fadd_rn(__fmul_rn(v1, bf16_hi(c[j])), __fmul_rn(o1, bf16_hi(sn[j])));
                }
            }
            out[j] = pack_bf16_pair(v0, v1);
        }
        reinterpret_cast<uint4 *>(dst)[g] = *reinterpret_cast<uint4 *>(out);
    }
}

} /* namespace h3q8 */
