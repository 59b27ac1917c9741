// nvtx_range.h — NVTX ranges around the host side of every collective and fused operator.
//
// Off unless TBV_NVTX=1 (one cached flag test per call).  With a tool attached (ncu --nvtx, a timeline
// profiler) every enqueue shows up as "tbv.<op> <bytes>B", so device work can be attributed to the call that
// launched it.  The reference has host-clock accumulators only (step4/libtbvcoll.cpp:114,205-209); this is the
// tool-facing counterpart of them.  nvtx3 is header-only and resolves its injection library lazily.
#pragma once
#include <nvtx3/nvToolsExt.h>
#include <stdio.h>
#include <stdlib.h>

namespace tbv {

inline bool nvtx_on() {
  static const bool on = [] {
    const char* e = getenv("TBV_NVTX");
    return e && atoi(e) != 0;
  }();
  return on;
}

struct NvtxRange {
  bool on;
  NvtxRange(const char* name, size_t bytes) : on(nvtx_on()) {
    if (on) {
      char buf[96];
      snprintf(buf, sizeof(buf), "%s %zuB", name, bytes);
      nvtxRangePushA(buf);
    }
  }
  ~NvtxRange() {
    if (on) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace tbv
