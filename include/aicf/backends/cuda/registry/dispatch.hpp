#pragma once
// The two free functions a binding layer calls (same mangled names and parameter lists as the reference's
// dispatch.hpp:12-26, so code compiled against either header links against either library).
//
// Common rules: `inputs` / `outputs` are arrays of borrowed descriptors (device pointers are not owned, nothing is
// allocated or freed on the caller's behalf), `attrs` is null or points at an AttrBlob, work is only enqueued on
// `stream` (no synchronisation). Result codes:
//   dispatch_v0        Ok | InvalidArgument (malformed call) | NotImplemented (no variant takes the operands) |
//                      whatever the chosen variant's launch returns
//   dispatch_by_id_v0  Ok | InvalidArgument (malformed call, attr schema mismatch, operands refused by the variant) |
//                      NotImplemented (no variant of `kind` carries `kernel_id`) | the variant's own result
#include <cstdint>
#include <cuda_runtime.h>

#include "aicf/backends/cuda/registry/op_kind.hpp"
#include "aicf/backends/cuda/registry/status.hpp"
#include "aicf/backends/cuda/registry/tensor_desc.hpp"

namespace aicf::cuda {

// Priority dispatch: variants of `kind` are tried in descending priority and the first whose supported() accepts the
// operands runs.
Status dispatch_v0(OpKind kind, const TensorDesc* inputs, int32_t num_inputs, TensorDesc* outputs,
                   int32_t num_outputs, const void* attrs, cudaStream_t stream);

// Decision-applied dispatch: exactly the variant registered under `kernel_id` runs, or nothing does.
Status dispatch_by_id_v0(OpKind kind, const char* kernel_id, const TensorDesc* inputs,
                         int32_t num_inputs, TensorDesc* outputs, int32_t num_outputs,
                         const void* attrs, cudaStream_t stream);

}  // namespace aicf::cuda
