// Device-side clock trace, built only with -DB200_TRACE (python -m triton_b200.trace).
// Selected threads of CTA 0 append (tag, clock64) pairs to a buffer that follows the status
// word, one region per traced thread; b200_trace_read copies it out.  The production build
// compiles the macros to nothing.
#pragma once

#ifdef B200_TRACE
namespace tb {
constexpr int kTraceRegions = 4, kTraceEvents = 4096, kTraceOffset = 4;  // offset: words after the status word
}
#define B200_TRACE_DECL unsigned trace_n_ = 0
#define B200_TRACE_EVENT(status, region, tag)                                                   \
  do {                                                                                          \
    if (blockIdx.x == 0 && trace_n_ < (unsigned)tb::kTraceEvents) {                             \
      unsigned* t_ = (status) + tb::kTraceOffset + (((region) * tb::kTraceEvents + trace_n_) << 1); \
      t_[0] = (tag);                                                                            \
      t_[1] = (unsigned)clock64();                                                              \
      ++trace_n_;                                                                               \
    }                                                                                           \
  } while (0)
#else
#define B200_TRACE_DECL
#define B200_TRACE_EVENT(status, region, tag)
#endif
