/* libts2ts_selftest -- test-only companion of libts2ts_attn.
 *
 * The attention kernels never spin forever: every mbarrier wait gives up after a bounded number of polls, records
 * a code in the plan's status word and lets the CTA drain (the reference has no counterpart: its kernels come from
 * PyTorch).  That path cannot be reached through the product entry points without breaking a kernel, so this
 * library holds one small kernel that waits, with a poll limit of a few thousand, on a barrier nothing arrives on.
 */
#ifndef TS2TS_SELFTEST_H_
#define TS2TS_SELFTEST_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Launches the kernel on `stream`.  `status` is a device int32 word that must be 0 (e.g. word 0 of a plan buffer):
 * the kernel stores 1000 + code there once its wait has run out, which ts2ts_read_status then reports.  `cycles`
 * (device, may be NULL) receives the SM clock cycles the two waits took.  0 < code < 1000.  Returns 0 when launched. */
int ts2ts_selftest_bounded_wait(int32_t* status, int32_t code, long long* cycles, void* stream);

/* Poll limit this library was compiled with. */
unsigned ts2ts_selftest_spin_limit(void);

#ifdef __cplusplus
}
#endif
#endif /* TS2TS_SELFTEST_H_ */
