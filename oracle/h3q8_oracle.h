/* TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's q8 linear
 * arithmetic, used as the checker for the CUDA path (tests, smoke check, and the
 * timed CPU baseline of the benchmark).  Nothing in the shipped library calls it.
 *
 * Every function cites the file:line of greg31337/h3cli it follows.  The int8
 * GEMMs of the reference exist only as Metal shaders, so the linear operators
 * below are restatements of shader arithmetic; the weight packer is additionally
 * pinned against the reference's own src/weights/q8.c compiled as-is
 * (oracle/_ref) and against the golden vectors of tests/metal_q8.c:21-34.
 *
 * Parity pins: packer, bf16 rounding, per-row quantiser, W8A16 per-group-64 and
 * W8A8 per-channel follow reference code.  W8A8 with per-K-group *weight* scales
 * has no reference implementation: "parity unpinned" beyond exact int32 group
 * sums combined in ascending group order (src/metal/shaders.metal:2701-2741).
 */
#ifndef H3Q8_ORACLE_H
#define H3Q8_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* src/metal/shaders.metal:11-19 (identical: src/cuda/cuda_kernels.cuh:8-10) */
float    h3o_bf16_to_f32(uint16_t bits);
uint16_t h3o_f32_to_bf16(float value);

/* src/weights/q8.c:6-19 with the group size as a parameter (reference: 64).
 * group == 0 means one group spanning the whole row (per-output-channel). */
int h3o_q8_layout(uint32_t rows, uint32_t columns, uint32_t group,
                  size_t *scale_offset, size_t *bytes);
/* src/weights/q8.c:26-56 */
int h3o_q8_pack_rows(const uint16_t *source, int8_t *weights, float *scales,
                     uint32_t rows, uint32_t columns, uint32_t group);

/* src/metal/shaders.metal:788-794: bf16(float(q) * scale[n, k/group]) */
void h3o_q8_dequant(const int8_t *weights, const float *scales, uint16_t *out,
                    uint32_t rows, uint32_t columns, uint32_t group);

/* src/metal/shaders.metal:1391-1460.  rows < dispatch_rows are padding rows
 * (zero bytes, scale 1).  clip is 1 except for the MLP-input experiments. */
void h3o_quantize_rows(const uint16_t *input, int8_t *output, float *scales,
                       uint32_t rows, uint32_t dispatch_rows, uint32_t columns,
                       float clip);

/* src/cuda/cuda_kernels.cuh:879-893 (tanh branch) on one bf16 value */
uint16_t h3o_gelu_tanh_bf16(uint16_t value);
/* src/cuda/cuda_kernels.cuh:973-986: bf16(float(res) + float(branch)*float(gate)) */
uint16_t h3o_gate_residual_bf16(uint16_t residual, uint16_t branch, uint16_t gate);

/* H3O_ACT_SWIGLU: weight (and bias) have 2*output_dim rows, gate rows first;
 * out = bf16(silu(bf16(gate)) * up), up kept in fp32 on the int8 path
 * (src/metal/shaders.metal:2269-2314) and rounded to bf16 on the bf16 / W8A16 path
 * (linear output stored as bf16, then src/cuda/cuda_kernels.cuh:1047-1059). */
enum { H3O_ACT_NONE = 0, H3O_ACT_GELU_TANH = 1, H3O_ACT_SWIGLU = 2 };
enum { H3O_MODE_BF16 = 0, H3O_MODE_W8A16 = 1, H3O_MODE_W8A8 = 2 };

/* One fused linear: out = epilogue(input x weight^T).  Mirrors the argument
 * block of the CUDA library's raw entry points so tests read alike.
 *   BF16  : weight bf16 [N,K]                        (src/cuda/gpu_cuda.cu:927-1005)
 *   W8A16 : weight int8 [N,K], weight_scales [N, ceil(K/group)]
 *           B = bf16(float(q)*scale), FP64 dot as tests/metal_q8.c:124-133,
 *           + float(bias), rounded to bf16  (src/metal/shaders.metal:820-856)
 *   W8A8  : input int8 [M,K] + input_scales [M]; int32 dot;
 *           bf16((float(acc)*in_scale[row])*w_scale[col])
 *           (src/metal/shaders.metal:2455-2465); with weight_group != 0 the
 *           per-group int32 sums are scaled and summed in fp32, g ascending.
 * The linear result is rounded to bf16 first; GELU-tanh and gate/residual are
 * then applied as separate bf16->bf16 operators, as the reference's unfused
 * chain does. */
typedef struct {
    uint32_t mode, rows, input_dim, output_dim;
    const void *input;
    const void *weight;
    const float *weight_scales;
    uint32_t weight_group;
    const float *input_scales;
    const uint16_t *bias, *gate, *residual;
    uint32_t activation;
    uint16_t *output;
    int32_t *accumulators; /* optional [M,N] int32 dump, W8A8 per-channel only */
    int fast;              /* 0: scalar spec (FP64 dot); 1: blocked fp32 OpenMP */
    uint32_t input_group;  /* W8A8: K elements per activation scale (input_scales [M, K/group]);
                              0 = per token.  src/metal/shaders.metal:2663-2742 (per-1024 FC2 scales) */
} h3o_linear_args;
int h3o_linear(const h3o_linear_args *args);

/* src/metal/shaders.metal:3390-3473 (h3_gate_adaln_quantize_int8_scalar): gate + residual,
 * RMS norm with the shader's 256-lane strided fma accumulation and tree reduction, AdaLN
 * modulation, per-row int8.  rsqrt is 1/sqrtf here (the GPU's is an approximation), so the
 * int8 bytes are compared within one step.  row_map may be NULL (class 0). */
void h3o_gate_adaln_quantize(const uint16_t *residual, const uint16_t *branch, const uint16_t *gate_modulation,
                             const uint32_t *row_map, const uint16_t *norm_weight, const uint16_t *norm_modulation,
                             uint16_t *gated_residual, uint16_t *normalized, int8_t *quantized, float *quantized_scales,
                             uint32_t rows, uint32_t padded_rows, uint32_t width, uint32_t slots, uint32_t gate_slot,
                             uint32_t shift_slot, uint32_t scale_slot, float epsilon);

/* src/cuda/cuda_kernels.cuh:988-1045 with grouped = 1 (columns [head, q|k|v, head_dim]):
 * per-head RMS norm of q and k (fmaf accumulation in dimension order), learned weight, rotary
 * embedding on dimensions [0, 2*rope_half); outputs [row, head, head_dim]. */
void h3o_grouped_qkv_rope(const uint16_t *qkv, const uint16_t *q_weight, const uint16_t *k_weight, const uint16_t *rope_cos,
                          const uint16_t *rope_sin, uint16_t *query, uint16_t *key, uint16_t *value, uint32_t sequence,
                          uint32_t heads, uint32_t head_dim, uint32_t rope_half, float epsilon);

int h3o_threads(void);
void h3o_set_threads(int count);   /* OpenMP threads of the blocked (timed) path */
#ifdef __cplusplus
}
#endif
#endif
