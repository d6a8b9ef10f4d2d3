/* Memory-bound helper kernels around the tcgen05 GEMM, plus a plain CUDA-core
 * linear used for shapes the TMA path cannot take (K not a multiple of 16, N
 * not a multiple of 8) and as an on-device cross-check.
 *
 * All of them are single-pass, coalesced, 16-byte-vectorised where the shape
 * allows, one CTA of 256 threads per row (or per 64x64 output tile for the
 * plain linear).  Rounding follows the reference bit for bit:
 *   per-token quantiser   src/metal/shaders.metal:1391-1460
 *   group weight packer   src/weights/q8.c:26-56
 *   weight dequantiser    src/metal/shaders.metal:788-794
 */
#pragma once
#include <float.h>
#include "gemm_tcgen05_pair_w8a16.cuh"

namespace h3q8 {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
/* max over a 256-thread CTA; every thread gets the result */
__device__ __forceinline__ float block_max_256(float v, float *scratch8) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch8[0];
#pragma unroll
    for (int i = 1; i < 8; i++) r = fmaxf(r, scratch8[i]);
    __syncthreads();
    return r;
}
/* Largest |x| of bf16 values as BIT PATTERNS.  For bf16, |a| <= |b| exactly when (a & 0x7fff) <= (b & 0x7fff) as
 * integers, and Inf / NaN are exactly the patterns >= 0x7f80: an integer maximum therefore carries a NaN to the end of
 * the reduction, where fmaxf would silently drop it (the reference rejects NaN and Inf alike, src/weights/q8.c:38-41,
 * tests/quant_native.c:64-74).  Two elements per instruction on packed pairs. */
__device__ __forceinline__ uint32_t absmax2(uint32_t running, uint32_t packed_pair) { return __vmaxu2(running, packed_pair & 0x7fff7fffu); }
__device__ __forceinline__ uint32_t absmax_fold(uint32_t packed) { return max(packed & 0xffffu, packed >> 16); }
__device__ __forceinline__ bool absmax_nonfinite(uint32_t folded) { return folded >= 0x7f80u; }
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
/* max over a 256-thread CTA; every thread gets the result */
__device__ __forceinline__ uint32_t block_max_256_u32(uint32_t v, uint32_t *scratch8) {
    v = warp_max_u32(v);
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    uint32_t r = scratch8[0];
#pragma unroll
    for (int i = 1; i < 8; i++) r = max(r, scratch8[i]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ int quantize_one(float x, float inverse) {
    int q = __float2int_rn(__fmul_rn(x, inverse)); /* rint: ties to even */
    return q < -127 ? -127 : q > 127 ? 127 : q;
}

/* Per-token (per-row) dynamic int8 quantiser.  Rows >= rows are padding: zero
 * bytes and scale 1.  One CTA per dispatched row.  Sets *nonfinite when a row
 * holds an Inf or a NaN. */
static __global__ void __launch_bounds__(256) quantize_rows_kernel(const uint16_t *__restrict__ in, int8_t *__restrict__ out,
                                                            float *__restrict__ scales, uint32_t rows, uint32_t columns,
                                                            float clip, uint32_t *nonfinite) {
    __shared__ uint32_t scratch[8];
    grid_dependency_trigger();   /* the GEMM that consumes these rows may set itself up while this grid drains */
    const uint32_t row = blockIdx.x;
    int8_t *q = out + (size_t)row * columns;
    const bool vec = (columns & 7u) == 0;
    if (row >= rows) {
        if (vec) for (uint32_t c = threadIdx.x; c < columns / 8; c += 256) reinterpret_cast<uint2 *>(q)[c] = make_uint2(0, 0);
        else for (uint32_t c = threadIdx.x; c < columns; c += 256) q[c] = 0;
        if (threadIdx.x == 0) scales[row] = 1.0f;
        return;
    }
    const uint16_t *x = in + (size_t)row * columns;
    uint32_t peak_bits = 0;
    uint4 held[2]; /* up to 4096 columns stay in registers between the two passes */
    const uint32_t vectors = columns / 8;
    if (vec) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            uint32_t c = threadIdx.x + i * 256;
            held[i] = c < vectors ? reinterpret_cast<const uint4 *>(x)[c] : make_uint4(0, 0, 0, 0);
            const uint32_t w[4] = {held[i].x, held[i].y, held[i].z, held[i].w};
#pragma unroll
            for (int j = 0; j < 4; j++) peak_bits = absmax2(peak_bits, w[j]);
        }
        for (uint32_t c = threadIdx.x + 512; c < vectors; c += 256) {
            uint4 v = reinterpret_cast<const uint4 *>(x)[c];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; j++) peak_bits = absmax2(peak_bits, w[j]);
        }
    } else {
        for (uint32_t c = threadIdx.x; c < columns; c += 256) peak_bits = absmax2(peak_bits, x[c]);
    }
    peak_bits = block_max_256_u32(absmax_fold(peak_bits), scratch);
    const float peak = bf16_bits_to_f32(peak_bits);
    const float clipped = __fmul_rn(peak, clip);
    const float scale = clipped > 0.0f ? __fdiv_rn(clipped, 127.0f) : __fdiv_rn(1.0f, 127.0f);
    const float inverse = clipped > 0.0f ? __fdiv_rn(127.0f, clipped) : 127.0f;
    if (threadIdx.x == 0) {
        scales[row] = scale;
        if (absmax_nonfinite(peak_bits) && nonfinite) atomicOr(nonfinite, STATUS_NONFINITE);
    }
    if (vec) {
        for (uint32_t c = threadIdx.x, i = 0; c < vectors; c += 256, i++) {
            uint4 v = i == 0 ? held[0] : i == 1 ? held[1] : reinterpret_cast<const uint4 *>(x)[c];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[2] = {0, 0};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t lo = (uint32_t)quantize_one(bf16_bits_to_f32(w[j] & 0xffffu), inverse) & 0xffu;
                uint32_t hi = (uint32_t)quantize_one(bf16_bits_to_f32(w[j] >> 16), inverse) & 0xffu;
                o[j >> 1] |= (lo | (hi << 8)) << ((j & 1) * 16);
            }
            reinterpret_cast<uint2 *>(q)[c] = make_uint2(o[0], o[1]);
        }
    } else {
        for (uint32_t c = threadIdx.x; c < columns; c += 256) q[c] = (int8_t)quantize_one(bf16_bits_to_f32(x[c]), inverse);
    }
}

/* The same quantiser with one WARP per segment (a row, or one K-group of a row) of at most
 * ITERS * 256 elements: every lane keeps its 16-byte vectors in registers between the maximum
 * and the rounding pass, nothing goes through shared memory and no CTA-wide barrier is
 * needed, so short segments (a 1024-wide group is 2 KB) keep many loads in flight.
 * Segment s covers in[s * segment ..); segments >= live are padding (zeros, scale 1). */
template <int ITERS>
static __global__ void __launch_bounds__(256) quantize_segments_warp_kernel(const uint16_t *__restrict__ in, int8_t *__restrict__ out,
                                                                     float *__restrict__ scales, uint64_t live, uint64_t total,
                                                                     uint32_t segment, float clip, uint32_t *nonfinite) {
    grid_dependency_trigger();   /* the GEMM that consumes these rows may set itself up while this grid drains */
    const uint64_t s = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (s >= total) return;
    const uint32_t lane = threadIdx.x & 31, vectors = segment / 8;
    uint2 *q = reinterpret_cast<uint2 *>(out + s * segment);
    if (s >= live) {
        for (uint32_t c = lane; c < vectors; c += 32) q[c] = make_uint2(0, 0);
        if (lane == 0) scales[s] = 1.0f;
        return;
    }
    const uint4 *x = reinterpret_cast<const uint4 *>(in + s * segment);
    uint4 held[ITERS];
    uint32_t peak_bits = 0;
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const uint32_t c = lane + i * 32;
        held[i] = c < vectors ? x[c] : make_uint4(0, 0, 0, 0);
        const uint32_t w[4] = {held[i].x, held[i].y, held[i].z, held[i].w};
#pragma unroll
        for (int j = 0; j < 4; j++) peak_bits = absmax2(peak_bits, w[j]);
    }
    peak_bits = warp_max_u32(absmax_fold(peak_bits));
    const float peak = bf16_bits_to_f32(peak_bits);
    const float clipped = __fmul_rn(peak, clip);
    const float scale = clipped > 0.0f ? __fdiv_rn(clipped, 127.0f) : __fdiv_rn(1.0f, 127.0f);
    const float inverse = clipped > 0.0f ? __fdiv_rn(127.0f, clipped) : 127.0f;
    if (lane == 0) {
        scales[s] = scale;
        if (absmax_nonfinite(peak_bits) && nonfinite) atomicOr(nonfinite, STATUS_NONFINITE);
    }
#pragma unroll
    for (int i = 0; i < ITERS; i++) {
        const uint32_t c = lane + i * 32;
        if (c >= vectors) break;
        const uint32_t w[4] = {held[i].x, held[i].y, held[i].z, held[i].w};
        uint32_t o[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t lo = (uint32_t)quantize_one(bf16_bits_to_f32(w[j] & 0xffffu), inverse) & 0xffu;
            uint32_t hi = (uint32_t)quantize_one(bf16_bits_to_f32(w[j] >> 16), inverse) & 0xffu;
            o[j >> 1] |= (lo | (hi << 8)) << ((j & 1) * 16);
        }
        q[c] = make_uint2(o[0], o[1]);
    }
}

/* Per-row (segment == columns) or per-K-group quantiser launch: the warp kernel when the segment is a
 * multiple of 8 of at most 4096 elements on 16-byte aligned rows, else one CTA per segment. */
static inline cudaError_t launch_quantize_rows(const uint16_t *in, int8_t *out, float *scales, uint64_t live, uint64_t total,
                                               uint32_t segment, float clip, uint32_t *nonfinite, cudaStream_t stream) {
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) & 15u) | (reinterpret_cast<uintptr_t>(out) & 7u)) == 0;
    const unsigned grid = (unsigned)((total + 7) / 8);
    if (aligned && segment % 8 == 0 && segment <= 1024)
        quantize_segments_warp_kernel<4><<<grid, 256, 0, stream>>>(in, out, scales, live, total, segment, clip, nonfinite);
    else if (aligned && segment % 8 == 0 && segment <= 3072)
        quantize_segments_warp_kernel<12><<<grid, 256, 0, stream>>>(in, out, scales, live, total, segment, clip, nonfinite);
    else if (aligned && segment % 8 == 0 && segment <= 4096)
        quantize_segments_warp_kernel<16><<<grid, 256, 0, stream>>>(in, out, scales, live, total, segment, clip, nonfinite);
    else
        quantize_rows_kernel<<<(unsigned)total, 256, 0, stream>>>(in, out, scales, (uint32_t)live, segment, clip, nonfinite);
    return cudaGetLastError();
}

/* Optional diagnostics of a quantisation (the job of quant_diagnostics, src/cuda/cuda_quant.cuh:72-87): a separate
 * scan, so the normal path pays nothing.  counts[0] += values whose magnitude exceeded the int8 range before clamping
 * (possible only with an activation clip below 1), counts[1] += non-zero values that became 0.  The scale of element
 * (r, c) is scales[r * groups + c / width]. */
static __global__ void __launch_bounds__(256) quant_diagnostics_kernel(const uint16_t *__restrict__ source, const int8_t *__restrict__ quantized,
                                                                      const float *__restrict__ scales, uint64_t rows, uint32_t columns,
                                                                      uint32_t width, uint32_t groups, unsigned long long *counts) {
    unsigned clipped = 0, zeroed = 0;
    const uint64_t total = rows * columns;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)blockDim.x * gridDim.x) {
        const uint64_t r = i / columns;
        const uint32_t c = (uint32_t)(i - r * columns);
        const float x = bf16_bits_to_f32(source[i]), scale = scales[r * groups + c / width];
        clipped += fabsf(__fdiv_rn(x, scale)) > 127.5f;
        zeroed += x != 0.0f && quantized[i] == 0;
    }
    if (clipped) atomicAdd(counts, (unsigned long long)clipped);
    if (zeroed) atomicAdd(counts + 1, (unsigned long long)zeroed);
}

/* Producer-side fusion of the activation quantiser (src/metal/shaders.metal:3390-3473,
 * src/gpu.h:630-642): per row
 *   gated = bf16(residual + branch * gate[class, gate_slot])          -> gated_residual (may alias residual)
 *   inv   = rsqrt(mean(gated^2) + epsilon)                             (fp32, fma accumulation, 256-way tree)
 *   v     = bf16(fma(gated * inv * norm_weight, 1 + scale[class], shift[class]))
 *   q     = per-row int8 of v (scale = max|v|/127)                    -> quantized, quantized_scales
 * so the W8A8 GEMM that follows reads int8 directly and the bf16 activation is never
 * re-read.  One 256-thread CTA per row; the row lives in shared memory between passes.
 * Rows in [rows, padded_rows) are written as zeros with scale 1.  HBM-bound:
 * 2*2*W read, 2*W + W + 4 written per row. */
static __global__ void __launch_bounds__(256) gate_adaln_quantize_kernel(
    const uint16_t *residual, const uint16_t *__restrict__ branch, const uint16_t *__restrict__ gate_modulation,
    const uint32_t *__restrict__ row_map, const uint16_t *__restrict__ norm_weight, const uint16_t *__restrict__ norm_modulation,
    uint16_t *gated_residual, int8_t *__restrict__ quantized, float *__restrict__ quantized_scales, uint32_t rows, uint32_t width,
    uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot, float epsilon, uint32_t *nonfinite) {
    extern __shared__ uint16_t row_values[];
    __shared__ float reductions[256];
    __shared__ uint32_t max_scratch[8];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const size_t row_base = (size_t)row * width;
    if (row >= rows) {
        for (uint32_t c = tid; c < width; c += 256) quantized[row_base + c] = 0;
        if (tid == 0) quantized_scales[row] = 1.0f;
        return;
    }
    const size_t base = (size_t)(row_map ? row_map[row] : 0) * slots * width;
    float local_sum = 0.0f;
    for (uint32_t c = tid; c < width; c += 256) {
        const float gate = bf16_bits_to_f32(gate_modulation[base + (size_t)gate_slot * width + c]);
        const uint32_t gated = f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(residual[row_base + c]),
                                                          __fmul_rn(bf16_bits_to_f32(branch[row_base + c]), gate)));
        gated_residual[row_base + c] = (uint16_t)gated;
        row_values[c] = (uint16_t)gated;
        const float v = bf16_bits_to_f32(gated);
        local_sum = fmaf(v, v, local_sum);
    }
    reductions[tid] = local_sum;
    __syncthreads();
    for (uint32_t stride = 128; stride >= 32; stride >>= 1) {
        if (tid < stride) reductions[tid] += reductions[tid + stride];
        __syncthreads();
    }
    if (tid < 32) {
        float sum = reductions[tid];
#pragma unroll
        for (int stride = 16; stride; stride >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, stride);
        if (tid == 0) reductions[0] = rsqrtf(__fadd_rn(__fdiv_rn(sum, (float)width), epsilon));
    }
    __syncthreads();
    const float inverse = reductions[0];
    uint32_t local_max = 0;
    for (uint32_t c = tid; c < width; c += 256) {
        const float normalized = __fmul_rn(__fmul_rn(bf16_bits_to_f32(row_values[c]), inverse), bf16_bits_to_f32(norm_weight[c]));
        const float shift = bf16_bits_to_f32(norm_modulation[base + (size_t)shift_slot * width + c]);
        const float scale = bf16_bits_to_f32(norm_modulation[base + (size_t)scale_slot * width + c]);
        const uint32_t v = f32_to_bf16_bits(fmaf(normalized, __fadd_rn(1.0f, scale), shift));   /* src/cuda/cuda_kernels.cuh:966-967 */
        row_values[c] = (uint16_t)v;
        local_max = absmax2(local_max, v & 0xffffu);
    }
    const uint32_t peak_bits = block_max_256_u32(absmax_fold(local_max), max_scratch);
    const float peak = bf16_bits_to_f32(peak_bits);
    if (tid == 0 && absmax_nonfinite(peak_bits) && nonfinite) atomicOr(nonfinite, STATUS_NONFINITE);
    const float out_scale = peak > 0.0f ? __fdiv_rn(peak, 127.0f) : __fdiv_rn(1.0f, 127.0f);
    const float q_scale = peak > 0.0f ? __fdiv_rn(127.0f, peak) : 127.0f;
    if (tid == 0) quantized_scales[row] = out_scale;
    for (uint32_t c = tid; c < width; c += 256) quantized[row_base + c] = (int8_t)quantize_one(bf16_bits_to_f32(row_values[c]), q_scale);
}

/* The same operator with one WARP per row: lane t plays the eight lanes 8t .. 8t+7 of the 256-lane reduction
 * (16-byte loads and stores, eight fma chains in the same element order), the tree steps 128/64/32/16/8 are shuffles
 * by 16/8/4/2/1 lanes and the steps 4/2/1 stay inside lane 0, so the sum is formed in exactly the same order, and no
 * CTA-wide barrier is needed.  The row is kept in the warp's own slice of shared memory between the three passes, not
 * in registers: with about 90 registers per thread five CTAs are resident per SM, and the operator, which is bound by
 * instruction issue and by its dependent passes rather than by HBM, lives on latency hiding (a register-resident
 * version ran at 0.57 / 0.34 of the HBM peak for widths 3072 / 5376, this one at 0.78 / 0.66).  Any width that is a
 * multiple of 8; dynamic shared memory = 4 warps x width x 2 bytes. */
static __global__ void __launch_bounds__(128) gate_adaln_quantize_warp_smem_kernel(
    const uint16_t *residual, const uint16_t *__restrict__ branch, const uint16_t *__restrict__ gate_modulation,
    const uint32_t *__restrict__ row_map, const uint16_t *__restrict__ norm_weight, const uint16_t *__restrict__ norm_modulation,
    uint16_t *gated_residual, int8_t *__restrict__ quantized, float *__restrict__ quantized_scales, uint32_t rows, uint32_t padded_rows,
    uint32_t width, uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot, float epsilon, uint32_t *nonfinite) {
    extern __shared__ uint4 row_store[];
    const uint32_t row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= padded_rows) return;
    const size_t row_base = (size_t)row * width;
    const uint32_t vectors = width / 8;
    uint4 *held = row_store + (threadIdx.x >> 5) * vectors;
    if (row >= rows) {
        for (uint32_t c = lane; c < vectors; c += 32) reinterpret_cast<uint2 *>(quantized + row_base)[c] = make_uint2(0, 0);
        if (lane == 0) quantized_scales[row] = 1.0f;
        return;
    }
    const size_t base = (size_t)(row_map ? row_map[row] : 0) * slots * width;
    const uint4 *res4 = reinterpret_cast<const uint4 *>(residual + row_base), *br4 = reinterpret_cast<const uint4 *>(branch + row_base);
    const uint4 *gate4 = reinterpret_cast<const uint4 *>(gate_modulation + base + (size_t)gate_slot * width);
    float sums[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    /* residual may alias gated_residual: the loads of four vectors are issued before any of their results is stored */
    for (uint32_t c0 = lane; c0 < vectors; c0 += 128) {
        uint4 r[4], b[4], g[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t c = c0 + k * 32;
            const bool live = c < vectors;
            r[k] = live ? res4[c] : make_uint4(0, 0, 0, 0);
            b[k] = live ? br4[c] : make_uint4(0, 0, 0, 0);
            g[k] = live ? gate4[c] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t c = c0 + k * 32;
            if (c < vectors) {
                const uint32_t rw[4] = {r[k].x, r[k].y, r[k].z, r[k].w}, bw[4] = {b[k].x, b[k].y, b[k].z, b[k].w};
                const uint32_t gw[4] = {g[k].x, g[k].y, g[k].z, g[k].w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    o[j] = pack_bf16_pair(__fadd_rn(bf16_lo(rw[j]), __fmul_rn(bf16_lo(bw[j]), bf16_lo(gw[j]))),
                                          __fadd_rn(bf16_hi(rw[j]), __fmul_rn(bf16_hi(bw[j]), bf16_hi(gw[j]))));
                    sums[2 * j] = fmaf(bf16_lo(o[j]), bf16_lo(o[j]), sums[2 * j]);
                    sums[2 * j + 1] = fmaf(bf16_hi(o[j]), bf16_hi(o[j]), sums[2 * j + 1]);
                }
                const uint4 gated = make_uint4(o[0], o[1], o[2], o[3]);
                held[c] = gated;
                reinterpret_cast<uint4 *>(gated_residual + row_base)[c] = gated;
            }
        }
    }
#pragma unroll
    for (int shift = 16; shift; shift >>= 1)
#pragma unroll
        for (int j = 0; j < 8; j++) sums[j] = __fadd_rn(sums[j], __shfl_down_sync(0xffffffffu, sums[j], shift));
    float sum = __fadd_rn(__fadd_rn(__fadd_rn(sums[0], sums[4]), __fadd_rn(sums[2], sums[6])),
                          __fadd_rn(__fadd_rn(sums[1], sums[5]), __fadd_rn(sums[3], sums[7])));
    const float inverse = __shfl_sync(0xffffffffu, rsqrtf(__fadd_rn(__fdiv_rn(sum, (float)width), epsilon)), 0);
    const uint4 *nw4 = reinterpret_cast<const uint4 *>(norm_weight);
    const uint4 *shift4 = reinterpret_cast<const uint4 *>(norm_modulation + base + (size_t)shift_slot * width);
    const uint4 *scale4 = reinterpret_cast<const uint4 *>(norm_modulation + base + (size_t)scale_slot * width);
    uint32_t local_max = 0;
#pragma unroll 2
    for (uint32_t c = lane; c < vectors; c += 32) {   /* each lane reads back only what it wrote itself */
        const uint4 n = nw4[c], sh = shift4[c], sc = scale4[c], own = held[c];
        const uint32_t vw[4] = {own.x, own.y, own.z, own.w}, nw[4] = {n.x, n.y, n.z, n.w};
        const uint32_t hw[4] = {sh.x, sh.y, sh.z, sh.w}, cw[4] = {sc.x, sc.y, sc.z, sc.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float n0 = __fmul_rn(__fmul_rn(bf16_lo(vw[j]), inverse), bf16_lo(nw[j]));
            const float n1 = __fmul_rn(__fmul_rn(bf16_hi(vw[j]), inverse), bf16_hi(nw[j]));
            /* one fused multiply-add, as the reference's CUDA build of this formula has it (src/cuda/cuda_kernels.cuh:966-967) */
            o[j] = pack_bf16_pair(fmaf(n0, __fadd_rn(1.0f, bf16_lo(cw[j])), bf16_lo(hw[j])),
                                  fmaf(n1, __fadd_rn(1.0f, bf16_hi(cw[j])), bf16_hi(hw[j])));
            local_max = absmax2(local_max, o[j]);
        }
        held[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    const uint32_t peak_bits = warp_max_u32(absmax_fold(local_max));
    const float peak = bf16_bits_to_f32(peak_bits);
    const float out_scale = peak > 0.0f ? __fdiv_rn(peak, 127.0f) : __fdiv_rn(1.0f, 127.0f);
    const float q_scale = peak > 0.0f ? __fdiv_rn(127.0f, peak) : 127.0f;
    if (lane == 0) {
        quantized_scales[row] = out_scale;
        if (absmax_nonfinite(peak_bits) && nonfinite) atomicOr(nonfinite, STATUS_NONFINITE);
    }
#pragma unroll 2
    for (uint32_t c = lane; c < vectors; c += 32) {
        const uint4 own = held[c];
        const uint32_t w[4] = {own.x, own.y, own.z, own.w};
        uint32_t o[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t lo = (uint32_t)quantize_one(bf16_lo(w[j]), q_scale) & 0xffu;
            uint32_t hi = (uint32_t)quantize_one(bf16_hi(w[j]), q_scale) & 0xffu;
            o[j >> 1] |= (lo | (hi << 8)) << ((j & 1) * 16);
        }
        reinterpret_cast<uint2 *>(quantized + row_base)[c] = make_uint2(o[0], o[1]);
    }
}

/* Weight-only Q8 group packer on the device: one warp per (row, K-group).
 * scale = max==0 ? 1 : max(max/127, FLT_MIN); q = round-half-even(w/scale). */
static __global__ void __launch_bounds__(256) q8_pack_rows_kernel(const uint16_t *__restrict__ src, int8_t *__restrict__ q,
                                                           float *__restrict__ scales, uint32_t rows, uint32_t columns,
                                                           uint32_t width, uint32_t groups, uint32_t *nonfinite) {
    const uint64_t item = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (uint64_t)rows * groups) return;
    const uint32_t row = (uint32_t)(item / groups), g = (uint32_t)(item % groups), lane = threadIdx.x & 31;
    const uint32_t first = g * width, last = columns - first < width ? columns : first + width;
    const uint16_t *x = src + (size_t)row * columns;
    uint32_t peak_bits = 0;
    for (uint32_t k = first + lane; k < last; k += 32) peak_bits = absmax2(peak_bits, x[k]);
    peak_bits = warp_max_u32(absmax_fold(peak_bits));
    const float peak = bf16_bits_to_f32(peak_bits);
    if (absmax_nonfinite(peak_bits) && lane == 0 && nonfinite) atomicOr(nonfinite, STATUS_NONFINITE);
    const float scale = peak == 0.0f ? 1.0f : fmaxf(__fdiv_rn(peak, 127.0f), FLT_MIN);
    if (lane == 0) scales[(size_t)row * groups + g] = scale;
    for (uint32_t k = first + lane; k < last; k += 32) {
        int v = __float2int_rn(__fdiv_rn(bf16_bits_to_f32(x[k]), scale));
        q[(size_t)row * columns + k] = (int8_t)(v < -127 ? -127 : v > 127 ? 127 : v);
    }
}

/* bf16(float(q) * scale[n, k/width]) for the whole matrix (dequant-to-scratch policy). */
static __global__ void __launch_bounds__(256) q8_dequant_kernel(const int8_t *__restrict__ q, const float *__restrict__ scales,
                                                         uint16_t *__restrict__ out, uint32_t rows, uint32_t columns,
                                                         uint32_t width, uint32_t groups) {
    grid_dependency_trigger();   /* a GEMM launched as a programmatic dependent may set itself up while this grid drains */
    const uint32_t row = blockIdx.y;
    const int8_t *src = q + (size_t)row * columns;
    uint16_t *dst = out + (size_t)row * columns;
    const float *s = scales + (size_t)row * groups;
    if ((columns & 15u) == 0 && (width & 15u) == 0) {
        for (uint32_t c = blockIdx.x * 256 + threadIdx.x; c < columns / 16; c += gridDim.x * 256) {
            const uint4 v = reinterpret_cast<const uint4 *>(src)[c];
            const float scale = s[(c * 16) / width];
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[8];
#pragma unroll
            for (int w = 0; w < 4; w++) {
                float f[4];
                dequant4(words[w], scale, f);
                o[2 * w] = pack_bf16x2(f[0], f[1]);
                o[2 * w + 1] = pack_bf16x2(f[2], f[3]);
            }
            reinterpret_cast<uint4 *>(dst)[2 * c] = make_uint4(o[0], o[1], o[2], o[3]);
            reinterpret_cast<uint4 *>(dst)[2 * c + 1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    } else {
        for (uint32_t c = blockIdx.x * 256 + threadIdx.x; c < columns; c += gridDim.x * 256)
            dst[c] = (uint16_t)f32_to_bf16_bits(__fmul_rn((float)src[c], s[c / width]));
    }
}

/* Plain CUDA-core linear with the same operand modes and epilogue as the
 * tcgen05 kernel: 64x64 output tile, 16x16 threads, 4x4 outputs per thread,
 * K slabs of 16 staged through shared memory as fp32 / int32. */
template <int MODE>
__global__ void __launch_bounds__(256) linear_plain_kernel(const void *__restrict__ xin, const void *__restrict__ win,
                                                           const GemmParams p) {
    using acc_t = typename std::conditional<MODE == MODE_W8A8, int32_t, float>::type;
    __shared__ acc_t xs[16][65];
    __shared__ acc_t ws[16][65];
    __shared__ acc_t ws2[16][65]; /* SwiGLU: the up-projection rows N + c of the same output columns */
    const bool swiglu = p.ep.activation == ACT_SWIGLU;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint32_t row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
    const uint32_t width = p.scale_group ? p.scale_group : p.K;
    const bool grouped8 = MODE == MODE_W8A8 && p.scale_group != 0;
    acc_t acc[4][4], acc2[4][4];
    float totals[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) { acc[i][j] = 0; acc2[i][j] = 0; totals[i][j] = 0.0f; }
    auto weight_value = [&](uint32_t wrow, uint32_t gk) -> acc_t {
        if (MODE == MODE_BF16) return (acc_t)bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(win)[(size_t)wrow * p.K + gk]);
        const int qv = reinterpret_cast<const int8_t *>(win)[(size_t)wrow * p.K + gk];
        if (MODE == MODE_W8A8) return (acc_t)qv;
        return (acc_t)bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn((float)qv, p.w_scales[(size_t)wrow * p.scale_groups + gk / width])));
    };
    for (uint32_t k0 = 0; k0 < p.K; k0 += 16) {
        for (uint32_t e = threadIdx.x; e < 64 * 16; e += 256) {
            const uint32_t r = e >> 4, k = e & 15;
            const uint32_t gr = row0 + r, gc = col0 + r, gk = k0 + k;
            acc_t xv = 0, wv = 0, wv2 = 0;
            if (gk < p.K) {
                if (gr < p.M) {
                    if (MODE == MODE_W8A8) xv = (acc_t)reinterpret_cast<const int8_t *>(xin)[(size_t)gr * p.K + gk];
                    else xv = (acc_t)bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(xin)[(size_t)gr * p.K + gk]);
                }
                if (gc < p.N) {
                    wv = weight_value(gc, gk);
                    if (swiglu) wv2 = weight_value(p.N + gc, gk);
                }
            }
            xs[k][r] = xv;
            ws[k][r] = wv;
            ws2[k][r] = wv2;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; k++) {
            acc_t a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = xs[k][ty * 4 + i]; b[i] = ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (MODE == MODE_W8A8) acc[i][j] += a[i] * b[j];
                    else acc[i][j] = (acc_t)fmaf((float)a[i], (float)b[j], (float)acc[i][j]);
                }
            if (swiglu) {
#pragma unroll
                for (int i = 0; i < 4; i++) b[i] = ws2[k][tx * 4 + i];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (MODE == MODE_W8A8) acc2[i][j] += a[i] * b[j];
                        else acc2[i][j] = (acc_t)fmaf((float)a[i], (float)b[j], (float)acc2[i][j]);
                    }
            }
        }
        __syncthreads();
        /* grouped W8A8: close the K-group -- scale its exact int32 sum and add in fp32 */
        if (grouped8 && ((k0 + 16) % width == 0 || k0 + 16 >= p.K)) {
            const uint32_t g = k0 / width;
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
                    if (r < p.M && c < p.N) {
                        float value = __fmul_rn(__fmul_rn((float)acc[i][j], p.a_scales[(size_t)r * p.a_scale_groups + (p.a_scale_groups == 1 ? 0 : g)]),
                                                p.w_scales[(size_t)c * p.scale_groups + (p.scale_groups == 1 ? 0 : g)]);
                        totals[i][j] = g ? __fadd_rn(totals[i][j], value) : value;
                    }
                    acc[i][j] = 0;
                }
        }
    }
    const bool gated = p.ep.gate != nullptr || p.ep.residual != nullptr;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
            if (r >= p.M || c >= p.N) continue;
            float linear;
            if (MODE == MODE_W8A8) {
                if (grouped8) linear = totals[i][j];
                else {
                    if (p.acc_dump) p.acc_dump[(size_t)r * p.N + c] = (int32_t)acc[i][j];
                    linear = __fmul_rn(__fmul_rn((float)acc[i][j], p.a_scales[r]), p.w_scales[c]);
                }
            } else {
                linear = (float)acc[i][j];
                if (p.acc_dump) {   /* fp32 partial sum */
                    p.acc_dump[(size_t)r * p.N + c] = __float_as_int(linear);
                    if (!p.out) continue;
                }
            }
            if (swiglu) { /* ungrouped scales only */
                float up = MODE == MODE_W8A8 ? __fmul_rn(__fmul_rn((float)acc2[i][j], p.a_scales[r]), p.w_scales[p.N + c]) : (float)acc2[i][j];
                if (p.ep.bias) { linear = __fadd_rn(linear, bf16_bits_to_f32(p.ep.bias[c])); up = __fadd_rn(up, bf16_bits_to_f32(p.ep.bias[p.N + c])); }
                p.out[(size_t)r * p.N + c] = (uint16_t)f32_to_bf16_bits(swiglu_f32(linear, up, MODE != MODE_W8A8));
                continue;
            }
            const uint32_t y = epilogue_value(linear, p.ep.bias ? bf16_bits_to_f32(p.ep.bias[c]) : 0.0f, p.ep.bias != nullptr,
                                              p.ep.activation, gated, p.ep.gate ? bf16_bits_to_f32(p.ep.gate[c]) : 1.0f,
                                              p.ep.residual ? bf16_bits_to_f32(p.ep.residual[(size_t)r * p.N + c]) : 0.0f);
            p.out[(size_t)r * p.N + c] = (uint16_t)y;
        }
}

} /* namespace h3q8 */
