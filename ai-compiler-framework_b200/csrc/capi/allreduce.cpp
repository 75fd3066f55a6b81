// Data-parallel gradient exchange: the all_reduce op (OpKind::AllReduce) and communicator set-up.
//
// One process per GPU. The communicator is process-global. NCCL is resolved at run time with
// dlopen("libnccl.so.2") so that a process which already loaded a NCCL (for instance through
// torch.distributed) shares that copy instead of mapping a second one; the library itself links
// only the CUDA runtime. Collectives are enqueued on the caller's stream and are legal under
// stream capture, so they become nodes of the captured train-step graph.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "aicf/backends/cuda/registry/kernel_variant.hpp"
#include "capi_internal.hpp"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok() const { return handle && GetUniqueId && CommInitRank && CommDestroy && AllReduce; }
};

NcclApi& nccl() {
  static NcclApi api = [] {
    NcclApi a;
    const char* override_path = std::getenv("AICF_NCCL_LIB");
    const char* names[] = {override_path, "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (!n || !n[0]) continue;
      a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.handle) break;
    }
    if (a.handle) {
      a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
      a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
      a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
      a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
      a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
    }
    return a;
  }();
  return api;
}

struct DpState {
  std::mutex mu;
  ncclComm_t comm = nullptr;
  int rank = 0;
  int world = 1;
};
DpState& dp() {
  static DpState s;
  return s;
}

int nccl_fail(ncclResult_t r, const char* what) {
  const char* txt = nccl().GetErrorString ? nccl().GetErrorString(r) : "?";
  return aicf::capi::fail(aicf::cuda::Status::Internal, std::string("[NCCL] ") + what + ": " + txt);
}

}  // namespace

namespace aicf::cuda {

namespace {

// inputs [G] -> outputs [G]; fp32, contiguous, same shape; in place when the pointers coincide.
bool all_reduce_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != DType::kF32 || out[0].dtype != DType::kF32) return false;
  if (!in[0].contiguous || !out[0].contiguous || in[0].rank() < 1) return false;
  if (in[0].rank() != out[0].rank()) return false;
  for (int i = 0; i < in[0].rank(); ++i)
    if (in[0].shape[i] != out[0].shape[i] || in[0].shape[i] <= 0) return false;
  return true;
}
bool all_reduce_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return all_reduce_check(in, ni, out, no);
}
Status all_reduce_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t,
                         cudaStream_t stream) {
  if (!all_reduce_check(in, ni, out, no)) return Status::InvalidArgument;
  const size_t n = static_cast<size_t>(in[0].numel());
  DpState& s = dp();
  if (s.world <= 1 || !s.comm) {
    // a single replica: the sum over ranks is the buffer itself
    if (in[0].data != out[0].data) {
      if (cudaMemcpyAsync(out[0].data, in[0].data, n * 4, cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
        cudaGetLastError();
        return Status::Internal;
      }
    }
    return Status::Ok;
  }
  const ncclResult_t r = nccl().AllReduce(in[0].data, out[0].data, n, ncclFloat32, ncclSum, s.comm, stream);
  return r == ncclSuccess ? Status::Ok : Status::Internal;
}
size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }

}  // namespace

KernelVariant make_all_reduce_nccl_f32_variant() {
  KernelVariant v{};
  v.name = "all_reduce_nccl_f32";
  v.flags = kKV_CaptureSafe;
  v.launch = all_reduce_launch;
  v.supported = all_reduce_supported;
  v.query_workspace = no_workspace;
  return v;
}

}  // namespace aicf::cuda

extern "C" {

int aicf_b200_dp_unique_id(void* id128) {
  if (!id128) return aicf::capi::fail(aicf::cuda::Status::InvalidArgument, "dp_unique_id: null buffer");
  if (!nccl().ok()) return aicf::capi::fail(aicf::cuda::Status::Internal, "dp: NCCL library not found (libnccl.so.2)");
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size is part of the ABI");
  ncclUniqueId id;
  const ncclResult_t r = nccl().GetUniqueId(&id);
  if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
  std::memcpy(id128, &id, sizeof(id));
  return AICF_OK;
}

int aicf_b200_dp_init(int rank, int world_size, const void* id128) {
  if (world_size < 1 || rank < 0 || rank >= world_size)
    return aicf::capi::fail(aicf::cuda::Status::InvalidArgument, "dp_init: bad rank/world_size");
  DpState& s = dp();
  std::lock_guard<std::mutex> lock(s.mu);
  if (s.comm) return aicf::capi::fail(aicf::cuda::Status::InvalidArgument, "dp_init: already initialised");
  if (world_size == 1) {
    s.rank = 0;
    s.world = 1;
    return AICF_OK;
  }
  if (!id128) return aicf::capi::fail(aicf::cuda::Status::InvalidArgument, "dp_init: null id");
  if (!nccl().ok()) return aicf::capi::fail(aicf::cuda::Status::Internal, "dp: NCCL library not found (libnccl.so.2)");
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  ncclComm_t comm = nullptr;
  const ncclResult_t r = nccl().CommInitRank(&comm, world_size, id, rank);
  if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
  s.comm = comm;
  s.rank = rank;
  s.world = world_size;
  return AICF_OK;
}

int aicf_b200_dp_finalize(void) {
  DpState& s = dp();
  std::lock_guard<std::mutex> lock(s.mu);
  if (s.comm) {
    nccl().CommDestroy(s.comm);
    s.comm = nullptr;
  }
  s.rank = 0;
  s.world = 1;
  return AICF_OK;
}

int aicf_b200_dp_world_size(void) { return dp().world; }
int aicf_b200_dp_rank(void) { return dp().rank; }

}  // extern "C"
