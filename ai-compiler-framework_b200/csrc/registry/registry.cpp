// Kernel registry and the two dispatch paths.
//
// Behaviour follows the reference's src/backends/cuda/registry/registry.cpp:
//   - by-id path (:16-64): unknown id -> NotImplemented, schema mismatch or supported()==false
//     -> InvalidArgument;
//   - legacy path (:144-195): first variant in descending priority (insertion order breaks ties)
//     whose schema gate and supported() pass, none -> NotImplemented.
// One deliberate difference: the reference returns NotImplemented whenever query_workspace() is
// non-zero (:52-56, :183-187). Here a scratch arena is handed to launch() instead.
#include "aicf/backends/cuda/registry/registry.hpp"

#include <atomic>
#include <cstdio>

#include "aicf/backends/cuda/nvtx.hpp"
#include "aicf/backends/cuda/registry/attr_blob.hpp"
#include "aicf/backends/cuda/registry/dispatch.hpp"
#include "aicf/backends/cuda/registry/register_all.hpp"

namespace aicf::cuda {

namespace {

// ---- dispatch scratch arena ------------------------------------------------------------------
// One arena per device, grown on demand, but never while the target stream is being captured (allocation is illegal
// there): a capture that needs more than is available gets no workspace.
// A block that has been handed to a launch is never freed or moved before the process exits: a CUDA graph captured
// earlier keeps the block's address inside its kernel nodes, so growing allocates a second, larger block and retires
// the first one in place. Growth is geometric, so the retired blocks together stay below the size of the live one.
// The arena is shared by every stream of its device: two launches that need workspace and are not ordered against
// each other (different streams, no event between them) use the same bytes. Callers that run such launches
// concurrently give each stream its own buffer through aicf_b200_launch_ws instead.
constexpr int kArenaDevices = 64;
struct DeviceArena {
  void* ptr = nullptr;
  size_t bytes = 0;
  std::vector<void*> retired;  // earlier blocks, kept alive for graphs that captured them
};
struct DispatchArena {
  std::mutex mu;
  void* user_ptr = nullptr;
  size_t user_bytes = 0;
  DeviceArena dev[kArenaDevices];
};
DispatchArena& arena() {
  static DispatchArena a;
  return a;
}
constexpr size_t kDefaultArenaBytes = size_t(64) << 20;

Status acquire_workspace(size_t need, cudaStream_t stream, void** ptr, size_t* bytes) {
  DispatchArena& a = arena();
  std::lock_guard<std::mutex> lock(a.mu);
  if (a.user_ptr) {
    if (need > a.user_bytes) return Status::InvalidArgument;
    *ptr = a.user_ptr;
    *bytes = a.user_bytes;
    return Status::Ok;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kArenaDevices) {
    cudaGetLastError();
    return Status::Internal;
  }
  DeviceArena& d = a.dev[dev];
  if (d.ptr && need <= d.bytes) {
    *ptr = d.ptr;
    *bytes = d.bytes;
    return Status::Ok;
  }
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess) {
    cudaGetLastError();
    return Status::Internal;
  }
  if (cs != cudaStreamCaptureStatusNone) return Status::Internal;  // cannot allocate under capture
  size_t want = need > kDefaultArenaBytes ? need : kDefaultArenaBytes;
  if (want < 2 * d.bytes) want = 2 * d.bytes;
  void* fresh = nullptr;
  if (cudaMalloc(&fresh, want) != cudaSuccess) {
    cudaGetLastError();
    want = need;  // the doubled size may not fit; the request itself might
    if (cudaMalloc(&fresh, want) != cudaSuccess) {
      cudaGetLastError();
      return Status::Internal;
    }
  }
  if (d.ptr) d.retired.push_back(d.ptr);
  d.ptr = fresh;
  d.bytes = want;
  *ptr = d.ptr;
  *bytes = d.bytes;
  return Status::Ok;
}

const AttrBlob* normalize_attrs(const void* attrs) {
  static const AttrBlob kEmpty{};
  return attrs ? static_cast<const AttrBlob*>(attrs) : &kEmpty;
}

bool call_is_sane(const OpCall& c) {
  if (c.num_inputs < 0 || c.num_outputs < 0) return false;
  if (c.num_inputs > 0 && !c.inputs) return false;
  if (c.num_outputs > 0 && !c.outputs) return false;
  const int k = static_cast<int>(c.kind);
  return k >= 0 && k < static_cast<int>(OpKind::_Count);
}

Status run_variant(const KernelVariant* v, const OpCall& c, const AttrBlob* attrs) {
  AICF_NVTX_RANGE(v->kernel_id);  // one range per dispatched launch, named by the kernel id (AICF_ENABLE_NVTX=1)
  void* ws = nullptr;
  size_t ws_bytes = 0;
  if (v->query_workspace) {
    const size_t need = v->query_workspace(c.inputs, c.num_inputs, attrs);
    if (need != 0) {
      // No arena to be had (a caller-provided one that is too small, or the first large request arriving while the
      // stream is capturing): the variant is still called, without workspace. Variants that can do without it run
      // their workspace-free form (the GEMM drops its split over K); the others refuse with InvalidArgument.
      if (!ok(acquire_workspace(need, c.stream, &ws, &ws_bytes))) {
        ws = nullptr;
        ws_bytes = 0;
      }
    }
  }
  return v->launch(c.inputs, c.num_inputs, c.outputs, c.num_outputs, attrs, ws, ws_bytes, c.stream);
}

Status DispatchById(const OpCall& call, const char* kernel_id) {
  KernelRegistry::ensure_registered();
  if (!kernel_id || !kernel_id[0]) return Status::InvalidArgument;
  if (!call_is_sane(call)) return Status::InvalidArgument;
  const AttrBlob* attrs = normalize_attrs(call.attrs);

  const KernelVariant* v = KernelRegistry::instance().find_by_id(call.kind, kernel_id);
  if (!v || !v->supported || !v->launch) return Status::NotImplemented;
  if (v->expected_attr_schema_id != 0 && attrs->schema_id != v->expected_attr_schema_id)
    return Status::InvalidArgument;
  if (!v->supported(call.inputs, call.num_inputs, call.outputs, call.num_outputs, attrs))
    return Status::InvalidArgument;
  return run_variant(v, call, attrs);
}

}  // namespace

void set_dispatch_workspace(void* ptr, size_t bytes) {
  DispatchArena& a = arena();
  std::lock_guard<std::mutex> lock(a.mu);
  a.user_ptr = ptr;
  a.user_bytes = ptr ? bytes : 0;
}

KernelRegistry& KernelRegistry::instance() {
  static KernelRegistry r;
  return r;
}

void KernelRegistry::ensure_registered() {
  static std::once_flag once;
  std::call_once(once, [] { aicf_cuda_register_all_kernels(); });
}

void KernelRegistry::register_kernel(OpKind kind, KernelVariant v) {
  const int k = static_cast<int>(kind);
  if (k < 0 || k >= kKinds) return;
  if (!v.kernel_id || !v.kernel_id[0]) return;

  std::lock_guard<std::mutex> lock(mu_);
  auto& vec = table_[k];
  // keep descending priority; equal priorities stay in registration order
  size_t pos = 0;
  while (pos < vec.size() && vec[pos]->priority >= v.priority) ++pos;
  auto it = vec.insert(vec.begin() + static_cast<std::ptrdiff_t>(pos), std::make_unique<KernelVariant>(v));
  by_id_[k].emplace(std::string((*it)->kernel_id), it->get());  // emplace keeps an existing id
}

const KernelVariant* KernelRegistry::find_by_id(OpKind kind, const char* kernel_id) const {
  const int k = static_cast<int>(kind);
  if (k < 0 || k >= kKinds || !kernel_id || !kernel_id[0]) return nullptr;
  std::lock_guard<std::mutex> lock(mu_);
  auto it = by_id_[k].find(kernel_id);
  return it == by_id_[k].end() ? nullptr : it->second;
}

void KernelRegistry::variants_snapshot(OpKind kind, std::vector<const KernelVariant*>& out) const {
  out.clear();
  const int k = static_cast<int>(kind);
  if (k < 0 || k >= kKinds) return;
  std::lock_guard<std::mutex> lock(mu_);
  out.reserve(table_[k].size());
  for (const auto& p : table_[k]) out.push_back(p.get());
}

Status Dispatch(const OpCall& call) {
  KernelRegistry::ensure_registered();
  if (!call_is_sane(call)) return Status::InvalidArgument;
  const AttrBlob* attrs = normalize_attrs(call.attrs);

  std::vector<const KernelVariant*> vars;
  KernelRegistry::instance().variants_snapshot(call.kind, vars);
  for (const KernelVariant* v : vars) {
    if (!v->supported || !v->launch) continue;
    if (v->expected_attr_schema_id != 0 && attrs->schema_id != v->expected_attr_schema_id) continue;
    if (!v->supported(call.inputs, call.num_inputs, call.outputs, call.num_outputs, attrs)) continue;
    return run_variant(v, call, attrs);
  }
  return Status::NotImplemented;
}

Status dispatch_v0(OpKind kind, const TensorDesc* inputs, int32_t num_inputs, TensorDesc* outputs,
                   int32_t num_outputs, const void* attrs, cudaStream_t stream) {
  OpCall c{};
  c.kind = kind;
  c.inputs = inputs;
  c.num_inputs = num_inputs;
  c.outputs = outputs;
  c.num_outputs = num_outputs;
  c.attrs = attrs;
  c.stream = stream;
  return Dispatch(c);
}

Status dispatch_by_id_v0(OpKind kind, const char* kernel_id, const TensorDesc* inputs,
                         int32_t num_inputs, TensorDesc* outputs, int32_t num_outputs,
                         const void* attrs, cudaStream_t stream) {
  OpCall c{};
  c.kind = kind;
  c.inputs = inputs;
  c.num_inputs = num_inputs;
  c.outputs = outputs;
  c.num_outputs = num_outputs;
  c.attrs = attrs;
  c.stream = stream;
  return DispatchById(c, kernel_id);
}

}  // namespace aicf::cuda
