/* The same layout report as `contract layout`, from THIS repository's include/h3q8.h; the two
 * outputs must be identical (tests/test_abi_cpu.py). */
#include "h3q8.h"
#include <stddef.h>
#include <stdio.h>
#define FIELD(name) printf("%s %zu\n", #name, offsetof(h3_gpu_stats, name))
int main(void) {
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
