/*
 * Bring-up additions to the aster_b200 C ABI.  They exist only in a library built with
 * -DB200_BRINGUP (`python -m aster_b200.build --bringup`): the default build exports none of
 * this and refuses the work-skipping values of b200_gemm_desc.reserved[0] (1 = the producer
 * signals without copying, 2 = the MMA warp commits without multiplying, 4 = skip the
 * tail-split exchange, 32 = the epilogue computes but does not store C, 64 = 16-byte stores
 * only), all of which make a launch return garbage and serve only to time parts of the kernel.
 */
#ifndef ASTER_B200_BRINGUP_H_
#define ASTER_B200_BRINGUP_H_

#include "aster_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Bring-up aid (no counterpart in the reference): with a device buffer of grid_ctas * 16
 * uint64 words attached, every CTA of the plan's launches records global-timer readings (ns)
 * of its milestones at [cta * 16 + slot]: 0 entry, 1 prologue done, 2 previous kernel of the
 * stream complete, 3 first copy issued, 4 first stage landed, 5 last MMA committed, 6 last
 * accumulator ready, 7 last epilogue done, 8 exit, 9..15 the MMAs of the CTA's first seven work
 * items committed (12 is then overwritten with the SM cycles of the last item's epilogue).  A
 * stamp itself costs about a microsecond.  NULL detaches. */
int b200_gemm_debug_timeline(b200_gemm_plan* plan, void* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* ASTER_B200_BRINGUP_H_ */
