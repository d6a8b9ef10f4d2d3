/* TEST INFRASTRUCTURE ONLY.  Host-pointer launchers around the reference's OWN CUDA
 * element kernels (greg31337/h3cli src/cuda/cuda_kernels.cuh), which this file includes
 * from where the reference tree lies (-I<reference>); nothing of it is copied here.
 * Built by oracle/Makefile into oracle/_ref/libh3_cuda_kernels_ref.so with the
 * reference's own nvcc flags (Makefile:117: -O3 -std=c++17 --fmad=false, compute_100),
 * so the -m gpu tests can compare this library's fused epilogues, the unfused
 * operators and the CPU restatement with what the reference itself computes on the
 * same GPU.  Launch shapes follow src/cuda/cuda_reference_wrappers.cuh:518, 557, 633,
 * 659, 678, 789 and src/cuda/gpu_cuda.cu:961-966, 1130.
 *
 * Every function takes HOST arrays, copies them to the current device, runs one
 * reference kernel and copies the result back; 1 = ok, 0 = CUDA error. */
#include <cuda_runtime.h>
#include <stdint.h>
#include <vector>

#include "src/cuda/cuda_kernels.cuh"

namespace {

struct Scratch {
    std::vector<void *> held;
    bool ok = true;
    ~Scratch() { for (void *p : held) cudaFree(p); }
    template <class T> T *up(const T *host, size_t count) {
        if (!host || !count) return nullptr;
        void *d = nullptr;
        if (cudaMalloc(&d, count * sizeof(T)) != cudaSuccess) { ok = false; return nullptr; }
        held.push_back(d);
        if (cudaMemcpy(d, host, count * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) ok = false;
        return static_cast<T *>(d);
    }
    template <class T> T *room(size_t count) {
        void *d = nullptr;
        if (cudaMalloc(&d, count * sizeof(T)) != cudaSuccess) { ok = false; return nullptr; }
        held.push_back(d);
        return static_cast<T *>(d);
    }
    template <class T> int down(T *host, const T *device, size_t count) {
        if (!ok || cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return 0;
        return cudaMemcpy(host, device, count * sizeof(T), cudaMemcpyDeviceToHost) == cudaSuccess;
    }
};

} /* namespace */

extern "C" int h3ref_gelu_bf16(const uint16_t *input, uint16_t *output, uint32_t elements, uint32_t approximate) {
    Scratch s;
    const ushort *in = s.up(input, elements);
    ushort *out = s.room<ushort>(elements);
    if (!s.ok) return 0;
    gelu_bf16_args args{elements, approximate};
    h3_gelu_bf16<<<dim3((elements + 255) / 256), dim3(256)>>>(in, out, args);
    return s.down(output, out, elements);
}

extern "C" int h3ref_gate_bf16(const uint16_t *residual, const uint16_t *branch, const uint16_t *modulation, const uint32_t *row_map,
                               uint16_t *output, uint32_t rows, uint32_t width, uint32_t slots, uint32_t gate_slot, uint32_t classes) {
    Scratch s;
    const size_t n = (size_t)rows * width;
    const ushort *r = s.up(residual, n), *b = s.up(branch, n), *m = s.up(modulation, (size_t)classes * slots * width);
    const uint *map = s.up(row_map, rows);
    ushort *out = s.room<ushort>(n);
    if (!s.ok) return 0;
    gate_args args{rows, width, slots, gate_slot};
    h3_gate_bf16<<<dim3((width + 15) / 16, (rows + 15) / 16), dim3(16, 16)>>>(r, b, m, map, out, args);
    return s.down(output, out, n);
}

extern "C" int h3ref_adaln_bf16(const uint16_t *input, const uint16_t *norm_weight, const uint16_t *modulation, const uint32_t *row_map,
                                uint16_t *output, uint32_t rows, uint32_t width, uint32_t slots, uint32_t shift_slot,
                                uint32_t scale_slot, float epsilon, uint32_t classes) {
    Scratch s;
    const size_t n = (size_t)rows * width;
    const ushort *x = s.up(input, n), *w = s.up(norm_weight, width), *m = s.up(modulation, (size_t)classes * slots * width);
    const uint *map = s.up(row_map, rows);
    ushort *out = s.room<ushort>(n);
    if (!s.ok) return 0;
    adaln_args args{rows, width, slots, shift_slot, scale_slot, epsilon};
    h3_adaln_bf16<<<dim3(rows), dim3(256)>>>(x, w, m, map, out, args);
    return s.down(output, out, n);
}

extern "C" int h3ref_rms_norm_bf16(const uint16_t *input, const uint16_t *weight, uint16_t *output, uint32_t rows, uint32_t width,
                                   float epsilon) {
    Scratch s;
    const size_t n = (size_t)rows * width;
    const ushort *x = s.up(input, n), *w = s.up(weight, width);
    ushort *out = s.room<ushort>(n);
    if (!s.ok) return 0;
    norm_args args{rows, width, epsilon};
    h3_rms_norm_bf16<<<dim3(rows), dim3(256)>>>(x, w, out, args);
    return s.down(output, out, n);
}

extern "C" int h3ref_qkv_rope_bf16(const uint16_t *qkv, const uint16_t *q_weight, const uint16_t *k_weight, const uint16_t *rope_cos,
                                   const uint16_t *rope_sin, uint16_t *query, uint16_t *key, uint16_t *value, uint32_t sequence,
                                   uint32_t heads, uint32_t head_dim, uint32_t rope_half, uint32_t grouped, float epsilon) {
    Scratch s;
    const size_t n = (size_t)sequence * heads * head_dim;
    const ushort *in = s.up(qkv, 3 * n), *qw = s.up(q_weight, head_dim), *kw = s.up(k_weight, head_dim);
    const ushort *c = s.up(rope_cos, (size_t)sequence * rope_half), *sn = s.up(rope_sin, (size_t)sequence * rope_half);
    ushort *q = s.room<ushort>(n), *k = s.room<ushort>(n), *v = s.room<ushort>(n);
    if (!s.ok) return 0;
    qkv_args args{sequence, heads, head_dim, rope_half, grouped, epsilon};
    h3_qkv_rope_bf16<<<dim3((head_dim + 7) / 8, (heads + 3) / 4, (sequence + 3) / 4), dim3(8, 4, 4)>>>(in, qw, kw, c, sn, q, k, v, args);
    return s.down(query, q, n) && s.down(key, k, n) && s.down(value, v, n);
}

extern "C" int h3ref_swiglu_bf16(const uint16_t *fused, uint16_t *output, uint32_t rows, uint32_t width) {
    Scratch s;
    const size_t n = (size_t)rows * width;
    const ushort *in = s.up(fused, 2 * n);
    ushort *out = s.room<ushort>(n);
    if (!s.ok) return 0;
    swiglu_args args{rows, width};
    h3_swiglu_bf16<<<dim3((width + 15) / 16, (rows + 15) / 16), dim3(16, 16)>>>(in, out, args);
    return s.down(output, out, n);
}

extern "C" int h3ref_add_bf16(const uint16_t *left, const uint16_t *right, uint16_t *output, uint32_t elements) {
    Scratch s;
    const ushort *l = s.up(left, elements), *r = s.up(right, elements);
    ushort *out = s.room<ushort>(elements);
    if (!s.ok) return 0;
    h3_add_bf16<<<dim3((elements + 255) / 256), dim3(256)>>>(l, r, out, elements);
    return s.down(output, out, elements);
}

/* The reference's small-shape bf16 linear (fp32 fmaf chain in k order, bias seeded into the accumulator). */
extern "C" int h3ref_linear_bf16(const uint16_t *input, const uint16_t *weight, const uint16_t *bias, uint16_t *output, uint32_t rows,
                                 uint32_t input_dim, uint32_t output_dim) {
    Scratch s;
    const ushort *x = s.up(input, (size_t)rows * input_dim), *w = s.up(weight, (size_t)output_dim * input_dim);
    const ushort *b = s.up(bias, bias ? output_dim : 0);
    ushort *out = s.room<ushort>((size_t)rows * output_dim);
    if (!s.ok) return 0;
    linear_args args{rows, input_dim, output_dim, bias ? 1u : 0u};
    h3_linear_bf16<<<dim3((output_dim + 15) / 16, (rows + 15) / 16), dim3(16, 16)>>>(x, w, b, out, args);
    return s.down(output, out, (size_t)rows * output_dim);
}
