/* Drop-in check of libh3q8 against the REFERENCE's own headers (greg31337/h3cli src/gpu.h and
 * src/weights/residency.h, found through -I<reference>; this file includes nothing of this
 * repository).  Style of the reference's tests/test_gpu_contract.c:
 *   - every symbol of the linear / quantisation / streaming path that src/gpu.h declares and
 *     libh3q8 exports is referenced through the reference's prototype and must link;
 *   - `contract layout` prints sizeof(h3_gpu_stats) and the offsets of the counters this
 *     path feeds, as the reference's compiler lays them out;
 *   - `contract run` (needs a B200) creates a context, runs one bf16 linear through the
 *     reference's prototypes and reads stats.linear_dispatches from the reference's struct.
 * Built by oracle/Makefile into oracle/_ref/abi_contract when the reference tree is present. */
#include "src/gpu.h"
#include "src/weights/residency.h"
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static void (*volatile contract[])(void) = {
    (void (*)(void))h3_gpu_create, (void (*)(void))h3_gpu_free, (void (*)(void))h3_gpu_cancel, (void (*)(void))h3_gpu_error,
    (void (*)(void))h3_gpu_get_stats, (void (*)(void))h3_gpu_backend_name, (void (*)(void))h3_gpu_has_int8_mlp,
    (void (*)(void))h3_gpu_profile_set_label, (void (*)(void))h3_gpu_profile_mark,
    (void (*)(void))h3_gpu_begin, (void (*)(void))h3_gpu_continue, (void (*)(void))h3_gpu_submit, (void (*)(void))h3_gpu_synchronize,
    (void (*)(void))h3_gpu_tensor_alloc, (void (*)(void))h3_gpu_tensor_contents, (void (*)(void))h3_gpu_tensor_new_f32,
    (void (*)(void))h3_gpu_tensor_new_bf16, (void (*)(void))h3_gpu_tensor_new_i8, (void (*)(void))h3_gpu_tensor_from_f32,
    (void (*)(void))h3_gpu_tensor_from_bf16, (void (*)(void))h3_gpu_tensor_from_u32, (void (*)(void))h3_gpu_tensor_free,
    (void (*)(void))h3_gpu_tensor_elements, (void (*)(void))h3_gpu_tensor_dtype, (void (*)(void))h3_gpu_tensor_read_f32,
    (void (*)(void))h3_gpu_tensor_read_bf16, (void (*)(void))h3_gpu_tensor_read_u32, (void (*)(void))h3_gpu_tensor_write_f32,
    (void (*)(void))h3_gpu_tensor_write_bf16, (void (*)(void))h3_gpu_tensor_write_bf16_range,
    (void (*)(void))h3_gpu_event_new, (void (*)(void))h3_gpu_event_record, (void (*)(void))h3_gpu_event_wait, (void (*)(void))h3_gpu_event_free,
    (void (*)(void))h3_gpu_tensor_load_bf16, (void (*)(void))h3_gpu_tensor_read_file_bf16, (void (*)(void))h3_gpu_tensor_stream_file_bf16,
    (void (*)(void))h3_gpu_plan_weights, (void (*)(void))h3_gpu_release_weight_cache, (void (*)(void))h3_gpu_should_retry_streaming,
    (void (*)(void))h3_gpu_linear_bf16, (void (*)(void))h3_gpu_quant_configure, (void (*)(void))h3_gpu_quant_load,
    (void (*)(void))h3_gpu_quantize_weight_int8, (void (*)(void))h3_gpu_linear_int8_bf16, (void (*)(void))h3_gpu_mlp_int8_bf16,
    (void (*)(void))h3_gpu_gate_adaln_quantize_int8, (void (*)(void))h3_gpu_linear_int8_head_major_bf16,
    (void (*)(void))h3_gpu_grouped_qkv_linear_rope_int8, (void (*)(void))h3_gpu_grouped_qkv_linear_rope_bf16,
    (void (*)(void))h3_gpu_grouped_qkv_rope_bf16, (void (*)(void))h3_gpu_gelu_bf16, (void (*)(void))h3_gpu_gate_bf16,
    (void (*)(void))h3_gpu_swiglu_bf16, (void (*)(void))h3_gpu_add_bf16,
    (void (*)(void))h3_weight_mode_name, (void (*)(void))h3_weight_options_read, (void (*)(void))h3_weight_options_equal,
    (void (*)(void))h3_weight_plan_build, (void (*)(void))h3_weight_retry_cap, (void (*)(void))h3_weight_packed_size,
};

#define FIELD(name) printf("%s %zu\n", #name, offsetof(h3_gpu_stats, name))

static int layout(void) {
    printf("sizeof %zu\n", sizeof(h3_gpu_stats));
    FIELD(q8_weights); FIELD(q8_dispatches); FIELD(q8_load_seconds); FIELD(allocated_bytes); FIELD(live_bytes);
    FIELD(peak_live_bytes); FIELD(tensor_allocations); FIELD(direct_dispatches); FIELD(submissions); FIELD(linear_dispatches);
    FIELD(h2d_bytes); FIELD(d2h_bytes); FIELD(d2d_bytes); FIELD(streamed_bytes); FIELD(resident_weight_bytes);
    FIELD(stream_slot_bytes); FIELD(resident_block_mask); FIELD(resident_blocks); FIELD(active_weight_blocks);
    FIELD(device_bytes); FIELD(pinned_bytes); FIELD(peak_pinned_bytes); FIELD(stream_stalls); FIELD(transfer_seconds);
    FIELD(stream_wait_seconds); FIELD(linear_seconds); FIELD(h2d_seconds); FIELD(d2h_seconds); FIELD(quant_conversion_seconds);
    FIELD(quant_clipped_values); FIELD(quant_zeroed_values); FIELD(quant_projection_dispatches); FIELD(quant_cache_hits);
    FIELD(quant_cache_misses); FIELD(native_scratch_bytes); FIELD(native_scratch_allocations); FIELD(native_scratch_reuses);
    FIELD(subblock_kernel_seconds);
    return 0;
}

#define CHECK(condition) do { if (!(condition)) { fprintf(stderr, "contract: %s failed (%s)\n", #condition, gpu ? h3_gpu_error(gpu) : error); return 1; } } while (0)

static int run(void) {
    char error[256] = {0};
    h3_gpu *gpu = h3_gpu_create(NULL, error, sizeof error);
    CHECK(gpu != NULL);
    enum { M = 130, K = 256, N = 264 };
    uint16_t *x = malloc(sizeof(uint16_t) * M * K), *w = malloc(sizeof(uint16_t) * N * K), *y = malloc(sizeof(uint16_t) * M * N);
    CHECK(x && w && y);
    for (int i = 0; i < M * K; i++) x[i] = 0x3f80;                       /* 1.0 */
    for (int i = 0; i < N * K; i++) w[i] = (i / K) % 2 ? 0x3f00 : 0xbf00;   /* +0.5 / -0.5 by output channel */
    h3_gpu_tensor *tx = h3_gpu_tensor_from_bf16(gpu, x, M * K), *tw = h3_gpu_tensor_from_bf16(gpu, w, N * K);
    h3_gpu_tensor *ty = h3_gpu_tensor_new_bf16(gpu, M * N);
    CHECK(tx && tw && ty);
    h3_gpu_stats before, after;
    CHECK(h3_gpu_get_stats(gpu, &before));
    CHECK(h3_gpu_begin(gpu));
    CHECK(h3_gpu_linear_bf16(gpu, ty, tx, tw, NULL, M, K, N));
    CHECK(h3_gpu_submit(gpu));
    CHECK(h3_gpu_get_stats(gpu, &after));
    CHECK(after.linear_dispatches == before.linear_dispatches + 1);
    CHECK(after.submissions == before.submissions + 1);
    CHECK(after.live_bytes >= (uint64_t)2 * (M * K + N * K + M * N));
    CHECK(after.mps_linear_dispatches == 0 && after.attention_dispatches == 0 && after.subblock_kernel_seconds == 0.0);
    CHECK(h3_gpu_tensor_read_bf16(ty, y, M * N));
    for (int i = 0; i < M * N; i++) CHECK(y[i] == ((i % N) % 2 ? 0x4300 : 0xc300));   /* +-128.0 exactly */
    CHECK(strstr(h3_gpu_backend_name(gpu), "cuda") != NULL);
    uint64_t scale, global, bytes;
    CHECK(h3_weight_packed_size(128, 256, 2, &scale, &global, &bytes) && scale == 128 * 256 && global == scale + 128 * 4 && bytes % 256 == 0);
    h3_gpu_tensor_free(tx); h3_gpu_tensor_free(tw); h3_gpu_tensor_free(ty);
    h3_gpu_free(gpu);
    free(x); free(w); free(y);
    printf("contract run ok: %zu symbols linked\n", sizeof contract / sizeof contract[0]);
    return 0;
}

int main(int argc, char **argv) {
    if (argc > 1 && !strcmp(argv[1], "layout")) return layout();
    if (argc > 1 && !strcmp(argv[1], "run")) return run();
    printf("%zu symbols\n", sizeof contract / sizeof contract[0]);
    return contract[0] == NULL;
}
