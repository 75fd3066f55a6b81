#pragma once
// Plugin ABI of one kernel variant (reference: kernel_variant.hpp:30-62, sizeof == 56).
//   supported()       cheap, side-effect free feasibility test; re-run inside launch()
//   query_workspace() bytes of scratch the launch needs. The reference refuses any
//                     non-zero answer; here the dispatcher or the plan supplies an arena.
//   launch()          only enqueues work on `stream`: no allocation, no synchronisation.
// `attr` always points at an AttrBlob (the dispatcher substitutes an empty one for null).
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "aicf/backends/cuda/registry/status.hpp"
#include "aicf/backends/cuda/registry/tensor_desc.hpp"

namespace aicf::cuda {

enum KernelVariantFlags : uint32_t {
  kKV_None = 0,
  kKV_CaptureSafe = 1u << 0,
};

struct KernelVariant {
  const char* name = nullptr;
  const char* kernel_id = nullptr;  // stable id used by the by-id dispatch path; mandatory
  int priority = 0;                 // higher is tried first by the legacy dispatch
  uint32_t flags = 0;
  uint32_t expected_attr_schema_id = 0;  // non-zero makes the schema mandatory

  Status (*launch)(const TensorDesc* inputs, int num_inputs, TensorDesc* outputs, int num_outputs,
                   const void* attr, void* workspace, size_t workspace_bytes,
                   cudaStream_t stream) = nullptr;

  size_t (*query_workspace)(const TensorDesc* inputs, int num_inputs, const void* attr) = nullptr;

  bool (*supported)(const TensorDesc* inputs, int num_inputs, const TensorDesc* outputs,
                    int num_outputs, const void* attr) = nullptr;
};

static_assert(sizeof(KernelVariant) == 56, "KernelVariant layout is ABI");

}  // namespace aicf::cuda
