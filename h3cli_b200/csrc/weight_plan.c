/* Resident-or-streamed planning for the DiT blocks' packed weights (host only).
 *
 * Semantics of h3cli's src/weights/residency.c:52-79: given the bytes of one block,
 * the set of active blocks (bit mask, at most 50), free device memory, a safety reserve
 * and the bytes that later allocations will need, decide between
 *   resident  every active block fits beside reserve + future allocations
 *   partial   two streaming slots are always paid first; as many leading active blocks
 *             as still fit stay resident, but never all of them
 *   stream    two slots only
 * Test-only knobs cap the resident count and the visible capacity so that the plans can be
 * exercised without large allocations (H3_TEST_CUDA_RESIDENT_BLOCKS, H3_TEST_CUDA_CAPACITY_BYTES,
 * H3_CUDA_TEST_MEMORY_BUDGET, H3_CUDA_WEIGHT_MODE). */
#include "h3q8.h"
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define MAX_BLOCKS 50

static int reject(char *error, size_t size, const char *why) {
    if (error && size) snprintf(error, size, "%s", why);
    return 0;
}
static int checked_add(uint64_t a, uint64_t b, uint64_t *out) {
    if (b > UINT64_MAX - a) return 0;
    *out = a + b;
    return 1;
}
static int checked_mul(uint64_t a, uint64_t b, uint64_t *out) {
    if (a && b > UINT64_MAX / a) return 0;
    *out = a * b;
    return 1;
}

const char *h3_weight_mode_name(int mode) {
    switch (mode) {
    case H3_WEIGHTS_RESIDENT: return "resident";
    case H3_WEIGHTS_STREAM: return "stream";
    default: return "auto";
    }
}

/* Halves a positive ceiling; reaches zero from 50 within seven steps, -1 once at zero. */
int h3_weight_retry_cap(unsigned count) { return count ? (int)((count - 1) / 2) : -1; }

static int read_cap(const char *name, uint64_t *value, char *error, size_t size) {
    const char *text = getenv(name);
    if (!text) return 1;
    if (*text < '0' || *text > '9') return reject(error, size, "invalid CUDA weight test cap");
    char *end = NULL;
    errno = 0;
    unsigned long long parsed = strtoull(text, &end, 10);
    if (errno || *end) return reject(error, size, "invalid CUDA weight test cap");
    *value = parsed;
    return 1;
}

int h3_weight_options_read(h3_weight_options *out, int force_stream, char *error, size_t size) {
    if (!out) return 0;
    memset(out, 0, sizeof *out);
    out->max_resident = -1;
    const char *mode = getenv("H3_CUDA_WEIGHT_MODE");
    if (mode && strcmp(mode, "auto")) {
        if (!strcmp(mode, "resident")) out->mode = H3_WEIGHTS_RESIDENT;
        else if (!strcmp(mode, "stream")) out->mode = H3_WEIGHTS_STREAM;
        else return reject(error, size, "CUDA weight mode must be auto, resident, or stream");
    }
    if (force_stream) {
        if (out->mode == H3_WEIGHTS_RESIDENT) return reject(error, size, "--ssd-streaming conflicts with CUDA resident weight mode");
        out->mode = H3_WEIGHTS_STREAM;
    }
    uint64_t blocks = MAX_BLOCKS;
    if (!read_cap("H3_TEST_CUDA_RESIDENT_BLOCKS", &blocks, error, size) || blocks > MAX_BLOCKS)
        return reject(error, size, "H3_TEST_CUDA_RESIDENT_BLOCKS must be 0..50");
    if (getenv("H3_TEST_CUDA_RESIDENT_BLOCKS")) out->max_resident = (int)blocks;
    return read_cap("H3_TEST_CUDA_CAPACITY_BYTES", &out->capacity_limit, error, size) &&
           read_cap("H3_CUDA_TEST_MEMORY_BUDGET", &out->allocation_limit, error, size);
}

int h3_weight_options_equal(const h3_weight_options *a, const h3_weight_options *b) {
    return a && b && a->mode == b->mode && a->max_resident == b->max_resident && a->capacity_limit == b->capacity_limit &&
           a->allocation_limit == b->allocation_limit;
}

int h3_weight_plan_build(h3_weight_plan *plan, h3_weight_options options, uint64_t active_mask, uint64_t block_bytes,
                         uint64_t available, uint64_t live, uint64_t future, uint64_t reserve, char *error, size_t size) {
    if (!plan || !active_mask || (active_mask >> MAX_BLOCKS) || !block_bytes || options.mode < H3_WEIGHTS_AUTO ||
        options.mode > H3_WEIGHTS_STREAM || options.max_resident < -1 || options.max_resident > MAX_BLOCKS)
        return reject(error, size, "invalid weight planner input");
    memset(plan, 0, sizeof *plan);
    plan->options = options;
    plan->active_mask = active_mask;
    plan->live_bytes = live;
    plan->future_bytes = future;
    plan->reserve_bytes = reserve;
    plan->block_bytes = block_bytes;
    for (unsigned bit = 0; bit < MAX_BLOCKS; bit++) plan->active_count += (active_mask >> bit) & 1u;
    if (options.capacity_limit) { /* the test capacity covers what is already live */
        uint64_t room = options.capacity_limit > live ? options.capacity_limit - live : 0;
        if (room < available) available = room;
    }
    plan->free_bytes = available;
    uint64_t committed, everything, two_slots;
    if (!checked_add(future, reserve, &committed) || !checked_mul(block_bytes, plan->active_count, &everything) ||
        !checked_mul(block_bytes, 2, &two_slots))
        return reject(error, size, "weight planner byte overflow");
    const int covered = available >= committed;
    const uint64_t budget = covered ? available - committed : 0;
    const int cap_allows_all = options.max_resident < 0 || (unsigned)options.max_resident >= plan->active_count;
    if (options.mode != H3_WEIGHTS_STREAM && cap_allows_all && covered && everything <= budget) {
        plan->resident_count = plan->active_count;
        plan->resident_mask = active_mask;
        plan->resident_bytes = everything;
        plan->effective_mode = H3_WEIGHTS_RESIDENT;
        return 1;
    }
    if (options.mode == H3_WEIGHTS_RESIDENT)
        return reject(error, size, "resident weights need more capacity than available after future allocations/reserve or test cap");
    if (!covered || two_slots > budget)
        return reject(error, size, "insufficient CUDA capacity even for two-slot streaming plus future allocations/reserve");
    plan->slot_bytes = two_slots;
    plan->effective_mode = H3_WEIGHTS_STREAM;
    uint64_t keep = (budget - two_slots) / block_bytes;
    if (keep >= plan->active_count) keep = plan->active_count - 1; /* streaming keeps at least one block streamed */
    if (options.max_resident >= 0 && keep > (unsigned)options.max_resident) keep = (unsigned)options.max_resident;
    if (options.mode == H3_WEIGHTS_STREAM) keep = 0;
    plan->resident_count = (unsigned)keep;
    plan->resident_bytes = keep * block_bytes;
    if (keep) plan->effective_mode = H3_WEIGHTS_AUTO; /* "auto" here means partially resident */
    for (unsigned bit = 0; keep && bit < MAX_BLOCKS; bit++)
        if (active_mask & (UINT64_C(1) << bit)) { plan->resident_mask |= UINT64_C(1) << bit; keep--; }
    return 1;
}
