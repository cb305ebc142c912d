// Optional in-kernel timeline (compiled only with -DHA_TIMELINE, never in the shipped library):
// every CTA stamps %globaltimer at kernel entry, after the grid-dependency wait and at exit; the
// minimum and maximum over the CTAs of each kernel land in a caller-provided buffer
// [kernel][event][min, max] of unsigned 64-bit nanoseconds. Used to see how the kernels of one
// decode step overlap under programmatic dependent launch.
#pragma once

#include <stdint.h>

namespace ha {

enum TimelineKernel { kTlHashDecode = 0, kTlScoreHist, kTlSelect, kTlGather, kTlMerge, kTlSelectPlan, kTlKernels };
enum TimelineEvent { kTlEntry = 0, kTlAfterWait, kTlExit, kTlMarkA, kTlMarkB, kTlMarkC, kTlEvents };

#ifdef HA_TIMELINE
// in constant memory: the pointer is read at every stamp, and a global-memory load there would put an L2 round
// trip (about half a microsecond) into the very path that is being timed
__constant__ unsigned long long* g_timeline = nullptr;

__device__ __forceinline__ void tl_mark(int kernel, int event) {
    if (g_timeline == nullptr || threadIdx.x != 0) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    unsigned long long* slot = g_timeline + (kernel * kTlEvents + event) * 2;
    atomicMin(slot, t);
    atomicMax(slot + 1, t);
}
#define HA_TL(kernel, event) ::ha::tl_mark(kernel, event)
#else
#define HA_TL(kernel, event) ((void)0)
#endif

}  // namespace ha
