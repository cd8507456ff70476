// Timestamps from inside a kernel — only in builds with -DTIS_TIMELINE, which
// `python -m tiny_inference_server_b200.kernels.microbench timeline` makes for itself; in every other build the
// macros below are empty and the parameter structs have no such member.
//
// Thread 0 of every CTA writes the global timer (ns) at a handful of named places into the buffer that the host
// announced for the next launch (tis_timeline_next): [CTA][TIS_TIMELINE_SLOTS].  A decode kernel of this library
// is a chain of latencies (the end of the kernel before -> the dependency wait -> the first bytes -> the loop ->
// the reduction over the cluster); the stamps say which link takes how long, across all CTAs of a launch and
// relative to the launch before.  Reading the timer and storing it costs ~0.1 us a stamp: compare the places,
// not the sum.
#pragma once

#ifdef TIS_TIMELINE
constexpr int TIS_TIMELINE_SLOTS = 12;
struct Timeline { unsigned long long* at; };            // null: this launch is not recorded
Timeline tis_timeline_take();                           // the buffer announced for the next launch (once)
__device__ __forceinline__ void tis_stamp(const Timeline& t, int slot, unsigned who) {
    if (t.at != nullptr && threadIdx.x == who) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        const size_t cta = blockIdx.x + (size_t)gridDim.x * (blockIdx.y + (size_t)gridDim.y * blockIdx.z);
        t.at[cta * TIS_TIMELINE_SLOTS + slot] = now;
    }
}
#define TIS_TIMELINE_MEMBER Timeline timeline;
#define TIS_TIMELINE_TAKE(p) (p).timeline = tis_timeline_take()
#define TIS_STAMP(p, slot) tis_stamp((p).timeline, (slot), 0u)
#define TIS_STAMP_BY(p, slot, who) tis_stamp((p).timeline, (slot), (who))
#else
#define TIS_TIMELINE_MEMBER
#define TIS_TIMELINE_TAKE(p) do {} while (0)
#define TIS_STAMP(p, slot) do {} while (0)
#define TIS_STAMP_BY(p, slot, who) do {} while (0)
#endif
