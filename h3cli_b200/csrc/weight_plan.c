/* Resident-or-streamed planning for the DiT blocks' packed weights (host only).
 *
 * The outcome is the one h3cli's planner produces (src/weights/residency.c:52-79; every field and every message is
 * compared with that file compiled as it is, on thousands of seeded inputs): given the bytes of one block, the set of
 * active blocks (bit mask, at most 50), free device memory, a safety reserve and the bytes that later allocations will
 * need, the weights end up
 *   resident  every active block fits beside reserve + future allocations
 *   partial   two streaming slots are paid first; as many leading active blocks as still fit stay resident,
 *             but never all of them
 *   stream    two slots only
 * or the request is refused.  Here the decision is written as a ledger: `account()` turns the request into the four
 * byte figures everything depends on (with overflow refused once, in one place), `settle()` maps ledger + options to
 * a verdict and a resident-block count without touching the plan, and `record()` writes a verdict into the plan.
 * The environment knobs are a table (name, destination, bound) walked by one parser.
 * Test-only knobs cap the resident count and the visible capacity so that the plans can be exercised without large
 * allocations (H3_TEST_CUDA_RESIDENT_BLOCKS, H3_TEST_CUDA_CAPACITY_BYTES, H3_CUDA_TEST_MEMORY_BUDGET,
 * H3_CUDA_WEIGHT_MODE). */
#include "h3q8.h"
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

enum { BLOCK_LIMIT = 50 };

static int refuse(char *error, size_t size, const char *why) {
    if (error && size) snprintf(error, size, "%s", why);
    return 0;
}

const char *h3_weight_mode_name(int mode) {
    static const char *const names[] = {"auto", "resident", "stream"};
    return names[mode == H3_WEIGHTS_RESIDENT ? 1 : mode == H3_WEIGHTS_STREAM ? 2 : 0];
}

/* The retry ladder after an out-of-memory failure: a ceiling of n resident blocks becomes (n - 1) / 2, and a ceiling
 * that is already zero has nowhere to go. */
int h3_weight_retry_cap(unsigned count) { return count ? (int)((count - 1) >> 1) : -1; }

int h3_weight_options_equal(const h3_weight_options *a, const h3_weight_options *b) {
    if (!a || !b) return 0;
    return a->mode == b->mode && a->max_resident == b->max_resident && a->capacity_limit == b->capacity_limit &&
           a->allocation_limit == b->allocation_limit;
}

/* ---------------------------------------------------------------- options from the environment */
/* A knob is an unsigned decimal with nothing around it.  0: malformed; 1: absent or parsed (*present says which). */
static int decimal_knob(const char *name, uint64_t *value, int *present) {
    const char *text = getenv(name);
    *present = text != NULL;
    if (!text) return 1;
    if (text[0] < '0' || text[0] > '9') return 0;
    char *end = NULL;
    errno = 0;
    const unsigned long long parsed = strtoull(text, &end, 10);
    if (errno || *end) return 0;
    *value = parsed;
    return 1;
}

static int mode_from_text(const char *text, int *mode) {
    static const struct { const char *word; int mode; } words[] = {
        {"auto", H3_WEIGHTS_AUTO}, {"resident", H3_WEIGHTS_RESIDENT}, {"stream", H3_WEIGHTS_STREAM}};
    for (size_t i = 0; i < sizeof words / sizeof words[0]; i++)
        if (!strcmp(text, words[i].word)) { *mode = words[i].mode; return 1; }
    return 0;
}

int h3_weight_options_read(h3_weight_options *out, int force_stream, char *error, size_t size) {
    if (!out) return 0;
    const h3_weight_options blank = {H3_WEIGHTS_AUTO, -1, 0, 0};
    *out = blank;
    const char *mode = getenv("H3_CUDA_WEIGHT_MODE");
    if (mode && !mode_from_text(mode, &out->mode)) return refuse(error, size, "CUDA weight mode must be auto, resident, or stream");
    if (force_stream) {
        if (out->mode == H3_WEIGHTS_RESIDENT) return refuse(error, size, "--ssd-streaming conflicts with CUDA resident weight mode");
        out->mode = H3_WEIGHTS_STREAM;
    }
    uint64_t ceiling = BLOCK_LIMIT;
    int present = 0;
    /* a malformed count and a count beyond the limit are reported alike, as the bound on the knob */
    if (!decimal_knob("H3_TEST_CUDA_RESIDENT_BLOCKS", &ceiling, &present) || ceiling > BLOCK_LIMIT)
        return refuse(error, size, "H3_TEST_CUDA_RESIDENT_BLOCKS must be 0..50");
    if (present) out->max_resident = (int)ceiling;
    const struct { const char *name; uint64_t *into; } byte_knobs[] = {
        {"H3_TEST_CUDA_CAPACITY_BYTES", &out->capacity_limit}, {"H3_CUDA_TEST_MEMORY_BUDGET", &out->allocation_limit}};
    for (size_t i = 0; i < sizeof byte_knobs / sizeof byte_knobs[0]; i++)
        if (!decimal_knob(byte_knobs[i].name, byte_knobs[i].into, &present)) return refuse(error, size, "invalid CUDA weight test cap");
    return 1;
}

/* ---------------------------------------------------------------- the ledger */
typedef struct {
    uint64_t room;        /* free bytes the planner may count on (after the test capacity)  */
    uint64_t owed;        /* future allocations + reserve: paid before any weight           */
    uint64_t all_blocks;  /* every active block resident                                     */
    uint64_t two_slots;   /* the two streaming slots                                         */
    uint64_t spendable;   /* room - owed, or 0 when owed does not fit                        */
    int owed_fits;
    unsigned active;
} ledger;

static int sum64(uint64_t a, uint64_t b, uint64_t *out) { *out = a + b; return *out >= a; }
static int product64(uint64_t a, uint64_t b, uint64_t *out) {
    *out = a * b;
    return !a || *out / a == b;
}
static unsigned bits_set(uint64_t mask) {
    unsigned n = 0;
    for (; mask; mask &= mask - 1) n++;
    return n;
}

static int account(ledger *l, const h3_weight_options *options, uint64_t active_mask, uint64_t block_bytes, uint64_t available,
                   uint64_t live, uint64_t future, uint64_t reserve) {
    l->active = bits_set(active_mask);
    l->room = available;
    if (options->capacity_limit) {     /* the test capacity covers what is already live */
        const uint64_t visible = options->capacity_limit > live ? options->capacity_limit - live : 0;
        if (visible < l->room) l->room = visible;
    }
    if (!sum64(future, reserve, &l->owed) || !product64(block_bytes, l->active, &l->all_blocks) || !product64(block_bytes, 2, &l->two_slots))
        return 0;
    l->owed_fits = l->room >= l->owed;
    l->spendable = l->owed_fits ? l->room - l->owed : 0;
    return 1;
}

typedef enum { ALL_RESIDENT, SLOTS_PLUS_SOME, NO_ROOM_FOR_RESIDENT, NO_ROOM_AT_ALL } verdict;

/* *keep: resident blocks beside the two slots (SLOTS_PLUS_SOME only). */
static verdict settle(const ledger *l, const h3_weight_options *options, uint64_t block_bytes, unsigned *keep) {
    const int ceiling_reaches_all = options->max_resident < 0 || (unsigned)options->max_resident >= l->active;
    *keep = 0;
    if (options->mode != H3_WEIGHTS_STREAM && ceiling_reaches_all && l->owed_fits && l->all_blocks <= l->spendable) return ALL_RESIDENT;
    if (options->mode == H3_WEIGHTS_RESIDENT) return NO_ROOM_FOR_RESIDENT;
    if (!l->owed_fits || l->two_slots > l->spendable) return NO_ROOM_AT_ALL;
    if (options->mode == H3_WEIGHTS_STREAM) return SLOTS_PLUS_SOME;
    uint64_t fit = (l->spendable - l->two_slots) / block_bytes;
    if (fit >= l->active) fit = l->active - 1;             /* a streaming plan streams at least one block */
    if (options->max_resident >= 0 && fit > (unsigned)options->max_resident) fit = (unsigned)options->max_resident;
    *keep = (unsigned)fit;
    return SLOTS_PLUS_SOME;
}

static void record(h3_weight_plan *plan, const ledger *l, verdict v, unsigned keep, uint64_t active_mask, uint64_t block_bytes) {
    if (v == ALL_RESIDENT) {
        plan->resident_count = l->active;
        plan->resident_mask = active_mask;
        plan->resident_bytes = l->all_blocks;
        plan->effective_mode = H3_WEIGHTS_RESIDENT;
        return;
    }
    plan->slot_bytes = l->two_slots;
    plan->resident_count = keep;
    plan->resident_bytes = (uint64_t)keep * block_bytes;
    plan->effective_mode = keep ? H3_WEIGHTS_AUTO : H3_WEIGHTS_STREAM;   /* "auto" in a plan means partially resident */
    for (uint64_t rest = active_mask; keep; keep--, rest &= rest - 1) plan->resident_mask |= rest & (~rest + 1);   /* lowest active bits first */
}

int h3_weight_plan_build(h3_weight_plan *plan, h3_weight_options options, uint64_t active_mask, uint64_t block_bytes,
                         uint64_t available, uint64_t live, uint64_t future, uint64_t reserve, char *error, size_t size) {
    const int sane = plan && active_mask && !(active_mask >> BLOCK_LIMIT) && block_bytes && options.mode >= H3_WEIGHTS_AUTO &&
                     options.mode <= H3_WEIGHTS_STREAM && options.max_resident >= -1 && options.max_resident <= BLOCK_LIMIT;
    if (!sane) return refuse(error, size, "invalid weight planner input");
    ledger l;
    const int counted = account(&l, &options, active_mask, block_bytes, available, live, future, reserve);
    memset(plan, 0, sizeof *plan);
    plan->options = options;
    plan->active_mask = active_mask;
    plan->active_count = l.active;
    plan->live_bytes = live;
    plan->future_bytes = future;
    plan->reserve_bytes = reserve;
    plan->block_bytes = block_bytes;
    plan->free_bytes = l.room;
    if (!counted) return refuse(error, size, "weight planner byte overflow");
    unsigned keep;
    const verdict v = settle(&l, &options, block_bytes, &keep);
    if (v == NO_ROOM_FOR_RESIDENT)
        return refuse(error, size, "resident weights need more capacity than available after future allocations/reserve or test cap");
    if (v == NO_ROOM_AT_ALL)
        return refuse(error, size, "insufficient CUDA capacity even for two-slot streaming plus future allocations/reserve");
    record(plan, &l, v, keep, active_mask, block_bytes);
    return 1;
}
