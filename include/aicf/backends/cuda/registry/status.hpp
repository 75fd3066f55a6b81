#pragma once
// Result codes returned by every dispatch entry point and kernel variant.
// Numeric values are ABI: they mirror the reference's
// include/aicf/backends/cuda/registry/status.hpp:6-11.
#include <cstdint>

namespace aicf::cuda {

enum class Status : int32_t { Ok = 0, InvalidArgument = 1, NotImplemented = 2, Internal = 3 };

// True for the one code that means the work was enqueued.
inline bool ok(Status s) { return s == Status::Ok; }

// Name of a code as it appears in error messages ("Unknown" for values outside the enum).
inline const char* status_to_string(Status s) {
  static const char* const kNames[] = {"Ok", "InvalidArgument", "NotImplemented", "Internal"};
  const int32_t i = static_cast<int32_t>(s);
  return (i >= 0 && i < 4) ? kNames[i] : "Unknown";
}

}  // namespace aicf::cuda
