// Diagnostic instrumentation of the contraction kernels, compiled in only with -DBAS_TRACE (a separate
// library built with `build.py --define BAS_TRACE --out ...`).  In the product build every macro below
// expands to nothing and the kernels carry no trace code.
//
//  * umma_colsplit_kernel: CTA 0 adds the cycles its roles spend waiting and working to a small device
//    array (GemmParams::trace) that bas_debug_trace() copies out, and stamps the global timer at the
//    start and end of every launch.
//  * umma_list_kernel: one chosen CTA stamps the global timer at eight events of each of the first
//    calls (ListParams::trace, read by bas_list_debug_trace()).
#pragma once

#ifdef BAS_TRACE
#define BAS_TRACE_ADD(slot, cycles) do { if (blockIdx.x == 0 && p.trace != nullptr) atomicAdd((unsigned long long*)&p.trace[slot], (unsigned long long)(cycles)); } while (0)
#define BAS_TRACE_CLOCK() clock64()
#define BAS_TRACE_SET(slot, v) do { if (blockIdx.x == 0 && p.trace != nullptr && (slot) < 512) p.trace[slot] = (long long)(v); } while (0)
// wall-clock start of CTA 0 of every launch (slots 300 + 2 * launch) and of every CTA of the latest one (600 + 2 * cta)
#define BAS_TRACE_LAUNCH_BEGIN()                                                          \
  int trace_launch = -1;                                                                  \
  if (blockIdx.x == 0 && threadIdx.x == 0 && p.trace != nullptr) {                        \
    trace_launch = (int)atomicAdd((unsigned long long*)&p.trace[30], 1ull);               \
    unsigned long long gt_;                                                               \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                               \
    if (trace_launch < 100) p.trace[300 + 2 * trace_launch] = (long long)gt_;             \
  }                                                                                       \
  if (threadIdx.x == 0 && p.trace != nullptr && blockIdx.x < 200) {                       \
    unsigned long long gt_;                                                               \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                               \
    p.trace[600 + 2 * blockIdx.x] = (long long)gt_;                                       \
  }
#define BAS_TRACE_LAUNCH_END()                                                            \
  if (trace_launch >= 0 && trace_launch < 100) {                                          \
    unsigned long long gt_;                                                               \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                               \
    p.trace[301 + 2 * trace_launch] = (long long)gt_;                                     \
  }                                                                                       \
  if (threadIdx.x == 0 && p.trace != nullptr && blockIdx.x < 200) {                       \
    unsigned long long gt_;                                                               \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                               \
    p.trace[601 + 2 * blockIdx.x] = (long long)gt_;                                       \
  }
// list kernel: [call][event] stamps of the chosen CTA
#define BAS_LTRACE_CALLS 256
#define BAS_LTRACE_EVENTS 8
#define BAS_LTRACE(call, ev)                                                                      \
  do {                                                                                            \
    if (p.trace != nullptr && blockIdx.x == p.trace_cta && (call) < BAS_LTRACE_CALLS) {           \
      unsigned long long gt_;                                                                     \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                                     \
      p.trace[(call) * BAS_LTRACE_EVENTS + (ev)] = (long long)gt_;                                \
    }                                                                                             \
  } while (0)
// second half of the array: issuer 0's tiles of a call, stamped when their data is seen (even slots) and
// when their MMAs have been issued (odd slots), the first four tiles of the call
#define BAS_LTRACE_TILE(call, k, phase)                                                           \
  do {                                                                                            \
    if (p.trace != nullptr && blockIdx.x == p.trace_cta && (call) < BAS_LTRACE_CALLS && (k) < 4) { \
      unsigned long long gt_;                                                                     \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                                     \
      p.trace[(BAS_LTRACE_CALLS + (call)) * BAS_LTRACE_EVENTS + 2 * (k) + (phase)] = (long long)gt_; \
    }                                                                                             \
  } while (0)
#else
#define BAS_TRACE_SET(slot, v) do { } while (0)
#define BAS_TRACE_ADD(slot, cycles) do { } while (0)
#define BAS_TRACE_CLOCK() 0LL
#define BAS_TRACE_LAUNCH_BEGIN() do { } while (0)
#define BAS_TRACE_LAUNCH_END() do { } while (0)
#define BAS_LTRACE(call, ev) do { } while (0)
#define BAS_LTRACE_TILE(call, k, phase) do { } while (0)
#endif
