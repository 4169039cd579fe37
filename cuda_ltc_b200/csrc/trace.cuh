// Optional per-warp event trace for the warp-specialised kernels (compiled in only with
// -DLTCA_TRACE; the shipped library contains none of it).  Lane 0 of every warp of ONE chosen
// CTA appends (tag, SM cycle counter) pairs to its own slice of a device buffer, which
// ltca_trace_read() copies out; the time line shows where each role waits.
#pragma once
#include <stdint.h>

#ifndef LTCA_TRACE_KERNEL
#define LTCA_TRACE_KERNEL 1   // which backward kernel records (1 = dQ, 2 = dK/dV)
#endif

#ifdef LTCA_TRACE
namespace ltca {
constexpr int kTraceWarps = 20;
constexpr int kTraceEvents = 2048;
static __device__ unsigned long long g_trace[kTraceWarps * kTraceEvents * 2];
static __device__ unsigned int g_trace_count[kTraceWarps];
struct TraceState {
    bool on;
    int n;
    __device__ __forceinline__ void init(bool cta_selected) {
        on = cta_selected && (threadIdx.x & 31) == 0;
        n = 0;
    }
    __device__ __forceinline__ void evt(uint32_t tag) {
        if (on && n < kTraceEvents) {
            const int w = threadIdx.x >> 5;
            unsigned long long t;
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
            g_trace[(w * kTraceEvents + n) * 2] = tag;
            g_trace[(w * kTraceEvents + n) * 2 + 1] = t;
            ++n;
            g_trace_count[w] = n;
        }
    }
};
}  // namespace ltca
#define LTCA_TRACE_DECL(sel) ::ltca::TraceState trace__; trace__.init(sel)
#define LTCA_TRACE_EVT(tag) trace__.evt(tag)
#else
#define LTCA_TRACE_DECL(sel) do { } while (0)
#define LTCA_TRACE_EVT(tag) do { } while (0)
#endif
