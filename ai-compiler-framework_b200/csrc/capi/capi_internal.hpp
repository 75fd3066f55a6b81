#pragma once
// Internals shared by the C ABI translation units.
#include <cuda_runtime.h>

#include <string>

#include "aicf/backends/cuda/registry/attr_blob.hpp"
#include "aicf/backends/cuda/registry/dispatch.hpp"
#include "aicf/backends/cuda/registry/registry.hpp"
#include "aicf_b200.h"

namespace aicf::capi {

void set_last_error(const std::string& msg);
int fail(aicf::cuda::Status st, const std::string& msg);
int check_cuda(cudaError_t e, const char* what);

inline cudaStream_t as_stream(aicf_stream s) { return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(s)); }
inline aicf_stream from_stream(cudaStream_t s) { return static_cast<aicf_stream>(reinterpret_cast<uintptr_t>(s)); }

inline const aicf::cuda::TensorDesc* as_desc(const aicf_tensor_desc* d) {
  return reinterpret_cast<const aicf::cuda::TensorDesc*>(d);
}
inline aicf::cuda::TensorDesc* as_desc(aicf_tensor_desc* d) { return reinterpret_cast<aicf::cuda::TensorDesc*>(d); }
inline const aicf::cuda::AttrBlob* as_blob(const aicf_attr_blob* b) {
  return reinterpret_cast<const aicf::cuda::AttrBlob*>(b);
}

}  // namespace aicf::capi
