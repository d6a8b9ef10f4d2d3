/* Host-side weight-only Q8 packer: bf16 [N,K] -> int8 [N,K] + fp32 scales per
 * K-group.  Behaviour of h3cli's src/weights/q8.c:6-56 (recipe 1: signed
 * symmetric groups along K, scale = max|w|/127 kept normal, round half to even,
 * clamp to +-127, non-finite input rejected), with the group width as a
 * parameter: 64 reproduces the reference layout, 128 is the DiT benchmark
 * layout, 0 means one scale per output channel. */
#include "h3q8.h"
#include <float.h>
#include <math.h>
#include <string.h>

static float bf16_value(uint16_t bits) {
    uint32_t word = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &word, sizeof value);
    return value;
}

int h3q8_q8_layout(uint32_t rows, uint32_t columns, uint32_t group, size_t *scale_offset, size_t *bytes) {
    if (!rows || !columns || !scale_offset || !bytes) return 0;
    const uint32_t width = group ? group : columns;
    if (columns > UINT32_MAX - (width - 1u)) return 0;
    const uint64_t elements = (uint64_t)rows * columns;
    if (elements > UINT32_MAX - 31u) return 0; /* kernels index weights with 32 bits */
    const uint64_t groups = ((uint64_t)columns + width - 1) / width;
    const uint64_t aligned = (elements + 3u) & ~(uint64_t)3u;
    const uint64_t total = aligned + rows * groups * sizeof(float);
    if (total > SIZE_MAX) return 0;
    *scale_offset = (size_t)aligned;
    *bytes = (size_t)total;
    return 1;
}

int h3q8_q8_pack_rows(const uint16_t *source, int8_t *weights, float *scales,
                      uint32_t rows, uint32_t columns, uint32_t group) {
    size_t offset, bytes;
    if (!source || !weights || !scales || !h3q8_q8_layout(rows, columns, group, &offset, &bytes)) return 0;
    const uint32_t width = group ? group : columns;
    const uint32_t groups = (uint32_t)(((uint64_t)columns + width - 1) / width);
    for (uint32_t n = 0; n < rows; n++) {
        const uint16_t *w = source + (size_t)n * columns;
        int8_t *q = weights + (size_t)n * columns;
        for (uint32_t g = 0; g < groups; g++) {
            const uint32_t begin = g * width;
            const uint32_t end = columns - begin < width ? columns : begin + width;
            float peak = 0.0f;
            for (uint32_t k = begin; k < end; k++) {
                const float v = bf16_value(w[k]);
                if (!isfinite(v)) return 0;
                peak = fmaxf(peak, fabsf(v));
            }
            const float scale = peak == 0.0f ? 1.0f : fmaxf(peak / 127.0f, FLT_MIN);
            scales[(size_t)n * groups + g] = scale;
            for (uint32_t k = begin; k < end; k++) {
                /* nearbyintf in the default rounding mode rounds halves to even */
                int v = (int)nearbyintf(bf16_value(w[k]) / scale);
                q[k] = (int8_t)(v < -127 ? -127 : v > 127 ? 127 : v);
            }
        }
    }
    return 1;
}

int h3_q8_layout(uint32_t rows, uint32_t columns, size_t *scale_offset, size_t *bytes) {
    return h3q8_q8_layout(rows, columns, H3_Q8_GROUP, scale_offset, bytes);
}

int h3_q8_pack_rows(const uint16_t *source, int8_t *weights, float *scales, uint32_t rows, uint32_t columns) {
    return h3q8_q8_pack_rows(source, weights, scales, rows, columns, H3_Q8_GROUP);
}
