// C entry points into the reference's own (unmodified) registry, compiled together with the
// reference sources where they lie by oracle/ref_build.py. TEST INFRASTRUCTURE: gives the GPU tests the
// reference's CUDA outputs on the same seeded inputs. Includes only the reference's public headers.
#include <cstdint>
#include <cuda_runtime.h>

#include "aicf/backends/cuda/registry/attr_blob.hpp"
#include "aicf/backends/cuda/registry/dispatch.hpp"
#include "aicf/backends/cuda/registry/op_kind.hpp"
#include "aicf/backends/cuda/registry/status.hpp"
#include "aicf/backends/cuda/registry/tensor_desc.hpp"

extern "C" {

int ref_tensor_desc_size() { return static_cast<int>(sizeof(aicf::cuda::TensorDesc)); }

int ref_op_call(int kind, const void* inputs, int num_inputs, void* outputs, int num_outputs, const void* attr_blob,
                uint64_t stream) {
  return static_cast<int>(aicf::cuda::dispatch_v0(
      static_cast<aicf::cuda::OpKind>(kind), static_cast<const aicf::cuda::TensorDesc*>(inputs), num_inputs,
      static_cast<aicf::cuda::TensorDesc*>(outputs), num_outputs, attr_blob,
      reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream))));
}

int ref_launch_by_id(const char* kernel_id, int kind, const void* inputs, int num_inputs, void* outputs,
                     int num_outputs, const void* attr_blob, uint64_t stream) {
  return static_cast<int>(aicf::cuda::dispatch_by_id_v0(
      static_cast<aicf::cuda::OpKind>(kind), kernel_id, static_cast<const aicf::cuda::TensorDesc*>(inputs), num_inputs,
      static_cast<aicf::cuda::TensorDesc*>(outputs), num_outputs, attr_blob,
      reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream))));
}

int ref_device_sync() { return static_cast<int>(cudaDeviceSynchronize()); }

}  // extern "C"
