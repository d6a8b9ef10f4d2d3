/* Declarations shared by the translation units of libh3q8 (not installed). */
#pragma once
#include <stdint.h>
namespace h3q8 {
int fail(const char *format, ...);      /* records the thread's error text, returns 0 */
void count_launch(unsigned kernels);    /* bumps the library-wide launch counter     */
uint32_t *device_status_word();         /* per-device error word, allocated on demand */
struct PairArgs;
/* grouped-scale two-CTA W8A8 kernel (its own translation unit, built with --fmad=false) */
int launch_pair_grouped_kernel(const PairArgs &args, bool magic, bool wide, int sms, void *stream);
}
