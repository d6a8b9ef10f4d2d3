/* TEST INFRASTRUCTURE ONLY -- see h3q8_oracle.h.  CPU restatement of the
 * reference's q8 linear arithmetic (greg31337/h3cli), used to check the CUDA
 * path and as the timed CPU baseline.  Compile with -ffp-contract=off: the
 * reference builds its CUDA with --fmad=false (Makefile:117) and writes every
 * formula as separate multiplies and adds. */
#include "h3q8_oracle.h"
#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int h3o_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* A launcher may have exported OMP_NUM_THREADS=1 (torch.distributed.run does); the timed CPU baseline asks for the
 * cores it is allowed to run on instead. */
void h3o_set_threads(int count) {
#ifdef _OPENMP
    if (count > 0) omp_set_num_threads(count);
#else
    (void)count;
#endif
}

/* src/metal/shaders.metal:11-13 */
float h3o_bf16_to_f32(uint16_t bits) {
    uint32_t word = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &word, 4);
    return value;
}

/* src/metal/shaders.metal:15-19: add 0x7fff plus the lsb of the kept half,
 * i.e. round to nearest even on the raw bits (NaN payloads are not special). */
uint16_t h3o_f32_to_bf16(float value) {
    uint32_t word;
    memcpy(&word, &value, 4);
    word += 0x7fffu + ((word >> 16) & 1u);
    return (uint16_t)(word >> 16);
}

static uint32_t group_width(uint32_t columns, uint32_t group) {
    return group ? group : columns;
}

/* src/weights/q8.c:6-19 */
int h3o_q8_layout(uint32_t rows, uint32_t columns, uint32_t group,
                  size_t *scale_offset, size_t *bytes) {
    uint32_t width = group_width(columns, group);
    if (!rows || !columns || !scale_offset || !bytes) return 0;
    if (columns > UINT32_MAX - (width - 1u)) return 0;
    uint64_t elements = (uint64_t)rows * columns;
    uint64_t groups = ((uint64_t)columns + width - 1) / width;
    if (elements > UINT32_MAX - 31u) return 0; /* 32-bit device indexing */
    uint64_t start = (elements + 3) & ~(uint64_t)3;
    uint64_t total = start + (uint64_t)rows * groups * sizeof(float);
    if (total > SIZE_MAX) return 0;
    *scale_offset = (size_t)start;
    *bytes = (size_t)total;
    return 1;
}

/* src/weights/q8.c:26-56.  Per row and K-group: scale = max|w|/127 clamped to
 * FLT_MIN (1 for an all-zero group); q = round-half-even(w/scale) clamped to
 * +-127.  nearbyintf under the default rounding mode is the same function as
 * the reference's floor/fraction/odd test for |w/scale| < 2^23. */
int h3o_q8_pack_rows(const uint16_t *source, int8_t *weights, float *scales,
                     uint32_t rows, uint32_t columns, uint32_t group) {
    size_t offset, bytes;
    if (!source || !weights || !scales ||
        !h3o_q8_layout(rows, columns, group, &offset, &bytes)) return 0;
    uint32_t width = group_width(columns, group);
    uint32_t groups = (uint32_t)(((uint64_t)columns + width - 1) / width);
    for (uint32_t n = 0; n < rows; n++) {
        const uint16_t *row = source + (size_t)n * columns;
        for (uint32_t g = 0; g < groups; g++) {
            uint32_t first = g * width;
            uint32_t last = columns - first < width ? columns : first + width;
            float peak = 0.0f;
            for (uint32_t k = first; k < last; k++) {
                float w = h3o_bf16_to_f32(row[k]);
                if (!isfinite(w)) return 0;
                peak = fmaxf(peak, fabsf(w));
            }
            float scale = peak == 0.0f ? 1.0f : fmaxf(peak / 127.0f, FLT_MIN);
            scales[(size_t)n * groups + g] = scale;
            for (uint32_t k = first; k < last; k++) {
                float ratio = h3o_bf16_to_f32(row[k]) / scale;
                float rounded = nearbyintf(ratio);
                int q = (int)rounded;
                if (q < -127) q = -127;
                if (q > 127) q = 127;
                weights[(size_t)n * columns + k] = (int8_t)q;
            }
        }
    }
    return 1;
}

/* src/metal/shaders.metal:788-794 */
void h3o_q8_dequant(const int8_t *weights, const float *scales, uint16_t *out,
                    uint32_t rows, uint32_t columns, uint32_t group) {
    uint32_t width = group_width(columns, group);
    uint32_t groups = (uint32_t)(((uint64_t)columns + width - 1) / width);
    for (uint32_t n = 0; n < rows; n++)
        for (uint32_t k = 0; k < columns; k++)
            out[(size_t)n * columns + k] = h3o_f32_to_bf16(
                (float)weights[(size_t)n * columns + k] *
                scales[(size_t)n * groups + k / width]);
}

/* src/metal/shaders.metal:1391-1460.  The stored scale is max/127 but the
 * quantiser multiplies by the separately computed inverse 127/max. */
void h3o_quantize_rows(const uint16_t *input, int8_t *output, float *scales,
                       uint32_t rows, uint32_t dispatch_rows, uint32_t columns,
                       float clip) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < dispatch_rows; r++) {
        int8_t *q = output + (size_t)r * columns;
        if (r >= rows) { /* :1402-1416 */
            memset(q, 0, columns);
            scales[r] = 1.0f;
            continue;
        }
        const uint16_t *x = input + (size_t)r * columns;
        float peak = 0.0f;
        for (uint32_t k = 0; k < columns; k++)
            peak = fmaxf(peak, fabsf(h3o_bf16_to_f32(x[k])));
        float clipped = peak * clip;
        float scale = clipped > 0.0f ? clipped / 127.0f : 1.0f / 127.0f;
        float inverse = clipped > 0.0f ? 127.0f / clipped : 127.0f;
        scales[r] = scale;
        for (uint32_t k = 0; k < columns; k++) {
            float scaled = h3o_bf16_to_f32(x[k]) * inverse;
            int v = (int)rintf(scaled);
            q[k] = (int8_t)(v < -127 ? -127 : v > 127 ? 127 : v);
        }
    }
}

/* src/cuda/cuda_kernels.cuh:883-893 */
uint16_t h3o_gelu_tanh_bf16(uint16_t bits) {
    float v = h3o_bf16_to_f32(bits);
    float cube = 0.044715f * v * v * v;
    float inner = 0.7978845608028654f * (v + cube);
    float activated;
    if (inner <= -10.0f) activated = 0.0f;
    else if (inner >= 10.0f) activated = v;
    else activated = 0.5f * v * (1.0f + tanhf(inner));
    return h3o_f32_to_bf16(activated);
}

/* src/cuda/cuda_kernels.cuh:979-984 */
uint16_t h3o_gate_residual_bf16(uint16_t residual, uint16_t branch, uint16_t gate) {
    float product = h3o_bf16_to_f32(branch) * h3o_bf16_to_f32(gate);
    float value = h3o_bf16_to_f32(residual) + product;
    return h3o_f32_to_bf16(value);
}

/* src/metal/shaders.metal:3390-3473 */
void h3o_gate_adaln_quantize(const uint16_t *residual, const uint16_t *branch, const uint16_t *gate_modulation,
                             const uint32_t *row_map, const uint16_t *norm_weight, const uint16_t *norm_modulation,
                             uint16_t *gated_residual, uint16_t *normalized_out, int8_t *quantized, float *quantized_scales,
                             uint32_t rows, uint32_t padded_rows, uint32_t width, uint32_t slots, uint32_t gate_slot,
                             uint32_t shift_slot, uint32_t scale_slot, float epsilon) {
    for (uint32_t row = 0; row < padded_rows; row++) {
        size_t row_base = (size_t)row * width;
        if (row >= rows) { /* :3405-3411 */
            memset(quantized + row_base, 0, width);
            quantized_scales[row] = 1.0f;
            continue;
        }
        size_t base = (size_t)(row_map ? row_map[row] : 0) * slots * width;
        float lanes[256];
        for (int t = 0; t < 256; t++) lanes[t] = 0.0f;
        for (uint32_t c = 0; c < width; c++) { /* :3419-3430, lane = c % 256 walks its columns in order */
            float gate = h3o_bf16_to_f32(gate_modulation[base + (size_t)gate_slot * width + c]);
            float product = h3o_bf16_to_f32(branch[row_base + c]) * gate;
            uint16_t gated = h3o_f32_to_bf16(h3o_bf16_to_f32(residual[row_base + c]) + product);
            gated_residual[row_base + c] = gated;
            float v = h3o_bf16_to_f32(gated);
            lanes[c % 256] = fmaf(v, v, lanes[c % 256]);
        }
        for (int stride = 128; stride >= 1; stride >>= 1) /* :3433-3444 */
            for (int t = 0; t < stride; t++) lanes[t] += lanes[t + stride];
        /* the reference calls rsqrt (shaders.metal:3446, cuda_kernels.cuh:957), which on a GPU is the hardware's
         * approximate instruction; a CPU has no bit-equal of it, so this restatement uses the correctly rounded value
         * and the GPU tests pin this operator against the reference's own CUDA kernels instead */
        float inverse = 1.0f / sqrtf(lanes[0] / (float)width + epsilon);
        float peak = 0.0f;
        for (uint32_t c = 0; c < width; c++) { /* :3450-3461 */
            float normalized = h3o_bf16_to_f32(gated_residual[row_base + c]) * inverse * h3o_bf16_to_f32(norm_weight[c]);
            float shift = h3o_bf16_to_f32(norm_modulation[base + (size_t)shift_slot * width + c]);
            float scale = h3o_bf16_to_f32(norm_modulation[base + (size_t)scale_slot * width + c]);
            uint16_t v = h3o_f32_to_bf16(fmaf(normalized, 1.0f + scale, shift)); /* one fused step: src/cuda/cuda_kernels.cuh:966-967 */
            normalized_out[row_base + c] = v;
            peak = fmaxf(peak, fabsf(h3o_bf16_to_f32(v)));
        }
        float out_scale = peak > 0.0f ? peak / 127.0f : 1.0f / 127.0f;
        float q_scale = peak > 0.0f ? 127.0f / peak : 127.0f;
        quantized_scales[row] = out_scale;
        for (uint32_t c = 0; c < width; c++) {
            int v = (int)rintf(h3o_bf16_to_f32(normalized_out[row_base + c]) * q_scale);
            quantized[row_base + c] = (int8_t)(v < -127 ? -127 : v > 127 ? 127 : v);
        }
    }
}

/* src/cuda/cuda_kernels.cuh:988-1045 */
void h3o_grouped_qkv_rope(const uint16_t *qkv, const uint16_t *q_weight, const uint16_t *k_weight, const uint16_t *rope_cos,
                          const uint16_t *rope_sin, uint16_t *query, uint16_t *key, uint16_t *value, uint32_t sequence,
                          uint32_t heads, uint32_t head_dim, uint32_t rope_half, float epsilon) {
#pragma omp parallel for schedule(static)
    for (uint32_t row = 0; row < sequence; row++)
        for (uint32_t head = 0; head < heads; head++) {
            size_t q_base = ((size_t)row * heads + head) * head_dim * 3, k_base = q_base + head_dim, v_base = k_base + head_dim;
            float q_sum = 0.0f, k_sum = 0.0f;
            for (uint32_t d = 0; d < head_dim; d++) {
                float q = h3o_bf16_to_f32(qkv[q_base + d]), k = h3o_bf16_to_f32(qkv[k_base + d]);
                q_sum = fmaf(q, q, q_sum);
                k_sum = fmaf(k, k, k_sum);
            }
            float qi = 1.0f / sqrtf(q_sum / (float)head_dim + epsilon), ki = 1.0f / sqrtf(k_sum / (float)head_dim + epsilon);
            for (uint32_t d = 0; d < head_dim; d++) {
                float q0 = h3o_bf16_to_f32(qkv[q_base + d]) * qi * h3o_bf16_to_f32(q_weight[d]);
                float k0 = h3o_bf16_to_f32(qkv[k_base + d]) * ki * h3o_bf16_to_f32(k_weight[d]);
                if (d < 2 * rope_half) {
                    int low = d < rope_half;
                    uint32_t pair = low ? d + rope_half : d - rope_half, first = low ? d : pair;
                    float q1 = h3o_bf16_to_f32(qkv[q_base + pair]) * qi * h3o_bf16_to_f32(q_weight[pair]);
                    float k1 = h3o_bf16_to_f32(qkv[k_base + pair]) * ki * h3o_bf16_to_f32(k_weight[pair]);
                    float c = h3o_bf16_to_f32(rope_cos[(size_t)row * rope_half + first]);
                    float s = h3o_bf16_to_f32(rope_sin[(size_t)row * rope_half + first]);
                    float qa = q0 * c, qb = q1 * s, ka = k0 * c, kb = k1 * s;
                    q0 = low ? qa - qb : qa + qb;
                    k0 = low ? ka - kb : ka + kb;
                }
                size_t o = ((size_t)row * heads + head) * head_dim + d;
                query[o] = h3o_f32_to_bf16(q0);
                key[o] = h3o_f32_to_bf16(k0);
                value[o] = qkv[v_base + d];
            }
        }
}

/* Everything after the linear result: bf16 round, then the reference's
 * separate bf16->bf16 operators in their call order. */
static float *capture; /* when set, receives the fp32 linear result (+bias) of every output */

static uint16_t finish(const h3o_linear_args *a, float linear, uint32_t r, uint32_t n) {
    if (a->bias) linear = linear + h3o_bf16_to_f32(a->bias[n]); /* shaders.metal:855 */
    if (capture) capture[(size_t)r * a->output_dim + n] = linear;
    uint16_t y = h3o_f32_to_bf16(linear);
    if (a->activation == H3O_ACT_GELU_TANH) y = h3o_gelu_tanh_bf16(y);
    if (a->residual || a->gate) {
        uint16_t one = 0x3f80, zero = 0;
        y = h3o_gate_residual_bf16(a->residual ? a->residual[(size_t)r * a->output_dim + n] : zero,
                                   y, a->gate ? a->gate[n] : one);
    }
    return y;
}

static int validate(const h3o_linear_args *a) {
    if (!a || !a->rows || !a->input_dim || !a->output_dim || !a->input ||
        !a->weight || !a->output) return 0;
    if (a->mode > H3O_MODE_W8A8) return 0;
    if (a->mode != H3O_MODE_BF16 && !a->weight_scales) return 0;
    if (a->mode == H3O_MODE_W8A8 && !a->input_scales) return 0;
    if (a->activation > H3O_ACT_SWIGLU) return 0;
    return 1;
}

/* Scalar specification.  W8A16 follows tests/metal_q8.c:124-133 (FP64 sum of
 * fp32 products of bf16 activations and bf16-rounded dequantised weights). */
static void linear_spec(const h3o_linear_args *a) {
    uint32_t M = a->rows, K = a->input_dim, N = a->output_dim;
    uint32_t chunk = a->weight_group ? a->weight_group : a->input_group;
    uint32_t width = group_width(K, a->mode == H3O_MODE_W8A8 ? chunk : a->weight_group);
    uint32_t groups = (uint32_t)(((uint64_t)K + width - 1) / width);
    uint32_t wgroups = a->weight_group ? groups : 1, agroups = a->input_group ? groups : 1;
#pragma omp parallel for schedule(dynamic, 4)
    for (uint32_t r = 0; r < M; r++) {
        for (uint32_t n = 0; n < N; n++) {
            float linear;
            if (a->mode == H3O_MODE_W8A8) {
                const int8_t *x = (const int8_t *)a->input + (size_t)r * K;
                const int8_t *w = (const int8_t *)a->weight + (size_t)n * K;
                if (!chunk) { /* shaders.metal:2455-2465 */
                    int32_t acc = 0;
                    for (uint32_t k = 0; k < K; k++) acc += (int32_t)x[k] * (int32_t)w[k];
                    if (a->accumulators) a->accumulators[(size_t)r * N + n] = acc;
                    linear = (float)acc * a->input_scales[r] * a->weight_scales[n];
                } else { /* shaders.metal:2701-2741 with the group scale on the weight */
                    linear = 0.0f;
                    for (uint32_t g = 0; g < groups; g++) {
                        int32_t acc = 0;
                        uint32_t last = (g + 1) * width < K ? (g + 1) * width : K;
                        for (uint32_t k = g * width; k < last; k++)
                            acc += (int32_t)x[k] * (int32_t)w[k];
                        float value = (float)acc * a->input_scales[(size_t)r * agroups + (agroups == 1 ? 0 : g)] *
                                      a->weight_scales[(size_t)n * wgroups + (wgroups == 1 ? 0 : g)];
                        linear = g ? linear + value : value;
                    }
                }
            } else {
                const uint16_t *x = (const uint16_t *)a->input + (size_t)r * K;
                double sum = 0.0;
                if (a->mode == H3O_MODE_W8A16) { /* shaders.metal:825-827 */
                    const int8_t *w = (const int8_t *)a->weight + (size_t)n * K;
                    const float *s = a->weight_scales + (size_t)n * groups;
                    for (uint32_t k = 0; k < K; k++) {
                        float b = h3o_bf16_to_f32(h3o_f32_to_bf16((float)w[k] * s[k / width]));
                        sum += (double)h3o_bf16_to_f32(x[k]) * (double)b;
                    }
                } else {
                    const uint16_t *w = (const uint16_t *)a->weight + (size_t)n * K;
                    for (uint32_t k = 0; k < K; k++)
                        sum += (double)h3o_bf16_to_f32(x[k]) * (double)h3o_bf16_to_f32(w[k]);
                }
                linear = (float)sum;
            }
            a->output[(size_t)r * N + n] = finish(a, linear, r, n);
        }
    }
}

/* Blocked fp32 / int32 version: the timed CPU baseline.  Same operand values
 * as the spec (bf16-rounded dequantised weights, exact int8 products); only
 * the fp32 summation order differs, so it is checked against the spec within
 * the bf16 tolerance and bit-exactly on the int32 path. */
#define RB 4   /* activation rows per micro-tile */
#define NB 64  /* output columns per micro-tile  */
#define KB 256 /* K slab kept in L1/L2           */

__attribute__((target_clones("avx512f", "avx2", "default")))
static void micro_f32(const float *x, size_t xs, const float *wt, uint32_t kb,
                      float acc[RB][NB]) {
    for (uint32_t k = 0; k < kb; k++) {
        const float *w = wt + (size_t)k * NB;
        for (int i = 0; i < RB; i++) {
            float xv = x[(size_t)i * xs + k];
            for (int j = 0; j < NB; j++) acc[i][j] += xv * w[j];
        }
    }
}

__attribute__((target_clones("avx512f", "avx2", "default")))
static void micro_i32(const int16_t *x, size_t xs, const int16_t *wt, uint32_t kb,
                      int32_t acc[RB][NB]) {
    for (uint32_t k = 0; k < kb; k++) {
        const int16_t *w = wt + (size_t)k * NB;
        for (int i = 0; i < RB; i++) {
            int32_t xv = x[(size_t)i * xs + k];
            for (int j = 0; j < NB; j++) acc[i][j] += xv * (int32_t)w[j];
        }
    }
}

static void linear_fast(const h3o_linear_args *a) {
    uint32_t M = a->rows, K = a->input_dim, N = a->output_dim;
    int integer = a->mode == H3O_MODE_W8A8;
    uint32_t chunk = a->weight_group ? a->weight_group : a->input_group;
    uint32_t width = group_width(K, integer ? chunk : a->weight_group);
    uint32_t groups = (uint32_t)(((uint64_t)K + width - 1) / width);
    uint32_t wgroups = a->weight_group ? groups : 1, agroups = a->input_group ? groups : 1;
    uint32_t kslab = integer && chunk ? width : KB;
    uint32_t ntiles = (N + NB - 1) / NB;
    /* Activations widened once: fp32 (bf16 is exact in fp32) or int16. */
    size_t xelements = (size_t)M * K;
    float *xf = integer ? NULL : malloc(xelements * sizeof(float));
    int16_t *xi = integer ? malloc(xelements * sizeof(int16_t)) : NULL;
    if (!xf && !xi) return;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < xelements; i++) {
        if (integer) xi[i] = ((const int8_t *)a->input)[i];
        else xf[i] = h3o_bf16_to_f32(((const uint16_t *)a->input)[i]);
    }
#pragma omp parallel
    {
        float *wtf = malloc((size_t)kslab * NB * sizeof(float));
        int16_t *wti = malloc((size_t)kslab * NB * sizeof(int16_t));
        float (*total)[NB] = malloc((size_t)M * sizeof(*total));
        int32_t (*itotal)[NB] = malloc((size_t)M * sizeof(*itotal));
#pragma omp for schedule(dynamic, 1)
        for (uint32_t t = 0; t < ntiles; t++) {
            uint32_t n0 = t * NB, nw = N - n0 < NB ? N - n0 : NB;
            memset(total, 0, (size_t)M * sizeof(*total));
            memset(itotal, 0, (size_t)M * sizeof(*itotal));
            for (uint32_t k0 = 0; k0 < K; k0 += kslab) {
                uint32_t kb = K - k0 < kslab ? K - k0 : kslab;
                /* transposed weight slab [kb][NB], dequantised as the spec does */
                for (uint32_t k = 0; k < kb; k++)
                    for (uint32_t j = 0; j < NB; j++) {
                        float wv = 0.0f;
                        int16_t wq = 0;
                        if (j < nw) {
                            size_t at = (size_t)(n0 + j) * K + k0 + k;
                            if (a->mode == H3O_MODE_BF16)
                                wv = h3o_bf16_to_f32(((const uint16_t *)a->weight)[at]);
                            else {
                                wq = ((const int8_t *)a->weight)[at];
                                if (!integer)
                                    wv = h3o_bf16_to_f32(h3o_f32_to_bf16((float)wq *
                                        a->weight_scales[(size_t)(n0 + j) * groups + (k0 + k) / width]));
                            }
                        }
                        wtf[(size_t)k * NB + j] = wv;
                        wti[(size_t)k * NB + j] = wq;
                    }
                uint32_t g = k0 / width;
                for (uint32_t r0 = 0; r0 < M; r0 += RB) {
                    uint32_t rw = M - r0 < RB ? M - r0 : RB;
                    if (!integer) {
                        float acc[RB][NB] = {{0}};
                        if (rw == RB) micro_f32(xf + (size_t)r0 * K + k0, K, wtf, kb, acc);
                        else for (uint32_t i = 0; i < rw; i++)
                            for (uint32_t k = 0; k < kb; k++)
                                for (uint32_t j = 0; j < NB; j++)
                                    acc[i][j] += xf[(size_t)(r0 + i) * K + k0 + k] * wtf[(size_t)k * NB + j];
                        for (uint32_t i = 0; i < rw; i++)
                            for (uint32_t j = 0; j < NB; j++) total[r0 + i][j] += acc[i][j];
                    } else {
                        int32_t acc[RB][NB] = {{0}};
                        if (rw == RB) micro_i32(xi + (size_t)r0 * K + k0, K, wti, kb, acc);
                        else for (uint32_t i = 0; i < rw; i++)
                            for (uint32_t k = 0; k < kb; k++)
                                for (uint32_t j = 0; j < NB; j++)
                                    acc[i][j] += (int32_t)xi[(size_t)(r0 + i) * K + k0 + k] * wti[(size_t)k * NB + j];
                        for (uint32_t i = 0; i < rw; i++)
                            for (uint32_t j = 0; j < nw; j++) {
                                if (!chunk) itotal[r0 + i][j] += acc[i][j];
                                else {
                                    float value = (float)acc[i][j] * a->input_scales[(size_t)(r0 + i) * agroups + (agroups == 1 ? 0 : g)] *
                                        a->weight_scales[(size_t)(n0 + j) * wgroups + (wgroups == 1 ? 0 : g)];
                                    total[r0 + i][j] = g ? total[r0 + i][j] + value : value;
                                }
                            }
                    }
                }
            }
            for (uint32_t r = 0; r < M; r++)
                for (uint32_t j = 0; j < nw; j++) {
                    float linear = total[r][j];
                    if (integer && !chunk) {
                        if (a->accumulators) a->accumulators[(size_t)r * N + n0 + j] = itotal[r][j];
                        linear = (float)itotal[r][j] * a->input_scales[r] * a->weight_scales[n0 + j];
                    }
                    a->output[(size_t)r * N + n0 + j] = finish(a, linear, r, n0 + j);
                }
        }
        free(wtf); free(wti); free(total); free(itotal);
    }
    free(xf); free(xi);
}

/* fc1 + SwiGLU: one linear over the [gate | up] rows, then the gated product. */
static int linear_swiglu(const h3o_linear_args *args) {
    uint32_t M = args->rows, N = args->output_dim;
    if (args->gate || args->residual || args->input_group) return 0;
    if (args->mode == H3O_MODE_W8A8 && args->weight_group) return 0; /* int8 SwiGLU: per-channel scales only */
    h3o_linear_args wide = *args;
    wide.output_dim = 2 * N;
    wide.activation = H3O_ACT_NONE;
    wide.accumulators = NULL;
    wide.output = malloc((size_t)M * 2 * N * sizeof(uint16_t));
    float *raw = malloc((size_t)M * 2 * N * sizeof(float));
    if (!wide.output || !raw) { free(wide.output); free(raw); return 0; }
    capture = raw;
    if (wide.fast) linear_fast(&wide); else linear_spec(&wide);
    capture = NULL;
    for (uint32_t r = 0; r < M; r++)
        for (uint32_t n = 0; n < N; n++) {
            float gate = h3o_bf16_to_f32(wide.output[(size_t)r * 2 * N + n]);
            float up = args->mode == H3O_MODE_W8A8 ? raw[(size_t)r * 2 * N + N + n]
                                                   : h3o_bf16_to_f32(wide.output[(size_t)r * 2 * N + N + n]);
            float value = gate / (1.0f + expf(-gate)) * up;
            args->output[(size_t)r * N + n] = h3o_f32_to_bf16(value);
        }
    free(wide.output);
    free(raw);
    return 1;
}

int h3o_linear(const h3o_linear_args *args) {
    if (!validate(args)) return 0;
    if (args->activation == H3O_ACT_SWIGLU) return linear_swiglu(args);
    if (args->fast) linear_fast(args);
    else linear_spec(args);
    return 1;
}
