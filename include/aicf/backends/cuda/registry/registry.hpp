#pragma once
// Kernel registry: per-OpKind priority-ordered variant table plus a by-id index
// (reference: registry.hpp:16-60, registry.cpp:66-142).
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>
#include <cuda_runtime.h>

#include "aicf/backends/cuda/registry/kernel_variant.hpp"
#include "aicf/backends/cuda/registry/op_kind.hpp"
#include "aicf/backends/cuda/registry/status.hpp"
#include "aicf/backends/cuda/registry/tensor_desc.hpp"

namespace aicf::cuda {

// One dispatch request. A plain aggregate passed by const reference; the field order and types are ABI (callers
// built against the reference's header fill it positionally or by name). All pointers are borrowed for the
// duration of the call; `attrs` is null or points at an AttrBlob whose payload dies when the call returns.
struct OpCall {
  OpKind kind{};
  const TensorDesc* inputs = nullptr;
  int32_t num_inputs = 0;
  TensorDesc* outputs = nullptr;
  int32_t num_outputs = 0;
  const void* attrs = nullptr;  // nullptr or AttrBlob*
  cudaStream_t stream = nullptr;
};

// Process-wide table of kernel variants. Only the member functions below are interface; callers never look inside
// the object (it lives in this library and is reached through instance()), so its private layout is free.
class KernelRegistry {
 public:
  // The one registry of the process (constructed on first use, never destroyed before exit).
  static KernelRegistry& instance();

  // Thread-safe. Variants without a kernel_id are ignored; the first registration of an id wins.
  void register_kernel(OpKind kind, KernelVariant v);

  // Stable pointers, taken under the lock so supported()/launch() run without it.
  void variants_snapshot(OpKind kind, std::vector<const KernelVariant*>& out) const;

  // The variant registered under `kernel_id` for `kind`, or null. The pointer stays valid for the life of the
  // process: variants are never removed.
  const KernelVariant* find_by_id(OpKind kind, const char* kernel_id) const;

  // Runs aicf_cuda_register_all_kernels() exactly once per process, whatever thread gets here first.
  static void ensure_registered();

 private:
  KernelRegistry() = default;
  static constexpr int kKinds = static_cast<int>(OpKind::_Count);
  // Per kind: variants in descending priority (ties in registration order), each owned here so that pointers
  // handed out by variants_snapshot / find_by_id never move, and an index from kernel id to variant.
  std::vector<std::unique_ptr<KernelVariant>> table_[kKinds];
  std::unordered_map<std::string, const KernelVariant*> by_id_[kKinds];
  mutable std::mutex mu_;  // guards both tables; never held while supported() or launch() run
};

// Legacy runtime dispatch: first supported variant in priority order.
Status Dispatch(const OpCall& call);

// Scratch arena used by dispatch for variants whose query_workspace() is non-zero: one lazily allocated block per
// device (64 MiB to start with, grown geometrically outside stream capture; outgrown blocks stay allocated because
// captured graphs may still point into them). The arena belongs to the device, not to a stream: launches that need
// workspace must be ordered against each other (same stream, or events between streams), or use
// aicf_b200_launch_ws with a buffer of their own.
// A caller-provided arena replaces the lazily allocated default (ptr == nullptr restores it).
void set_dispatch_workspace(void* ptr, size_t bytes);

}  // namespace aicf::cuda
