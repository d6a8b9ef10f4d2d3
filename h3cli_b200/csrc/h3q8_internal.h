/* Declarations shared by the translation units of libh3q8 (not installed). */
#pragma once
#include <stdint.h>
namespace h3q8 {
int fail(const char *format, ...);      /* records the thread's error text, returns 0 */
void count_launch(unsigned kernels);    /* bumps the library-wide launch counter     */
uint32_t *device_status_word();         /* per-device error word, allocated on demand */
uint32_t static_status_take();          /* error word inside the static scratch of h3q8_linear_w8a8_static, read and cleared */
struct PairArgs;
/* grouped-scale two-CTA W8A8 kernel (its own translation unit; every fp32 step is an explicit __fmul_rn / __fadd_rn) */
int launch_pair_grouped_kernel(const PairArgs &args, bool magic, bool wide, int sms, void *stream);
struct SkinnyArgs;
/* weight-streaming kernel for at most 64 rows: K split over a cluster, partial sums reduced through distributed shared memory */
int launch_skinny_kernel(SkinnyArgs &args, uint32_t mode, int sms, void *stream);
}
