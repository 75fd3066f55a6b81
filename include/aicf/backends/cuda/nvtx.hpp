#pragma once
// NVTX ranges around op launches (reference: include/aicf/backends/cuda/nvtx.hpp:16-37, AICF_NVTX_RANGE / NvtxRange,
// switched by the CMake option AICF_ENABLE_NVTX). Here the ranges are always compiled in - NVTX 3 is header-only and
// costs one predictable branch when no tool is attached - and switched at run time: AICF_ENABLE_NVTX=1 in the
// environment (read once per process) turns them on. A range covers the host-side enqueue of one op; under stream
// capture that is the moment the op's node is recorded, so a timeline tool shows which op produced which graph node.
#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

namespace aicf::cuda {

inline bool nvtx_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("AICF_ENABLE_NVTX");
    return e != nullptr && e[0] != '\0' && e[0] != '0';
  }();
  return on;
}

struct NvtxRange {
  explicit NvtxRange(const char* msg) : active_(nvtx_enabled()) {
    if (active_) nvtxRangePushA(msg ? msg : "aicf");
  }
  ~NvtxRange() {
    if (active_) nvtxRangePop();
  }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;

 private:
  bool active_;
};

}  // namespace aicf::cuda

#define AICF_NVTX_CONCAT_(a, b) a##b
#define AICF_NVTX_CONCAT(a, b) AICF_NVTX_CONCAT_(a, b)
#define AICF_NVTX_RANGE(MSG) ::aicf::cuda::NvtxRange AICF_NVTX_CONCAT(aicf_nvtx_range_, __LINE__)(MSG)
