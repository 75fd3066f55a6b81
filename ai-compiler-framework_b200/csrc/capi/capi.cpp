// C ABI: dispatch, registry introspection, op trace, the process-global CUDA graph and the
// device-memory helpers. Declarations and the reference interfaces they replace: include/aicf_b200.h.
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <deque>
#include <mutex>
#include <vector>

#include "capi_internal.hpp"

namespace aicf::cuda {
int gemm_tcgen05_status(bool clear);
int row_pipeline_status(bool clear);
int layernorm_pipeline_status(bool clear);
int adam_pipeline_status(bool clear);
int gemm_tcgen05_timeline(int enable, unsigned long long* out16);
void gemm_reload_env_overrides();
int dp_wait_status(bool clear);
Status stream_probe(int reads, int writes, const void* const* in, void* const* out, size_t bytes, int in_flight,
                    int blocks_per_sm, cudaStream_t stream);
}

static_assert(sizeof(aicf_tensor_desc) == sizeof(aicf::cuda::TensorDesc), "C and C++ tensor descriptors must match");
static_assert(offsetof(aicf_tensor_desc, dtype) == 8 && offsetof(aicf_tensor_desc, rank) == 12 &&
                  offsetof(aicf_tensor_desc, shape) == 16 && offsetof(aicf_tensor_desc, stride) == 48 &&
                  offsetof(aicf_tensor_desc, contiguous) == 80 && offsetof(aicf_tensor_desc, alignment) == 84 &&
                  offsetof(aicf_tensor_desc, device) == 88,
              "C tensor descriptor layout");
static_assert(sizeof(aicf_attr_blob) == sizeof(aicf::cuda::AttrBlob), "C and C++ attr blobs must match");

namespace aicf::capi {

namespace {
thread_local std::string t_last_error;
}

void set_last_error(const std::string& msg) { t_last_error = msg; }
int fail(aicf::cuda::Status st, const std::string& msg) {
  t_last_error = msg;
  return static_cast<int>(st);
}
int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return AICF_OK;
  t_last_error = std::string("[CUDA] ") + what + ": " + cudaGetErrorString(e);
  cudaGetLastError();
  return AICF_INTERNAL;
}

namespace {

using aicf::cuda::KernelRegistry;
using aicf::cuda::KernelVariant;
using aicf::cuda::OpKind;
using aicf::cuda::Status;

// ---- trace + graph share one mutex, as in the reference binding ---------------------------------
std::mutex g_mu;
std::deque<std::string> g_trace;
bool g_trace_on = true;
std::string g_trace_scratch;

void trace_push_locked(std::string s) {
  if (!g_trace_on) return;
  if (g_trace.size() >= AICF_B200_TRACE_CAPACITY) g_trace.pop_front();
  g_trace.push_back(std::move(s));
}

struct GraphState {
  bool capturing = false;
  bool captured = false;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaStream_t stream = nullptr;

  void drop_graph() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    exec = nullptr;
    graph = nullptr;
    captured = false;
  }
  // Ends a capture left dangling by an earlier failure, then drops any instantiated graph.
  void reset() {
    if (stream) {
      cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone) {
        cudaGraph_t tmp = nullptr;
        if (cudaStreamEndCapture(stream, &tmp) == cudaSuccess && tmp) cudaGraphDestroy(tmp);
      }
      cudaGetLastError();
    }
    drop_graph();
    capturing = false;
  }
};
GraphState g_graph;

std::string fail_text(int kind, Status st, const char* kernel_id) {
  std::string m = "aicf_cuda call failed: kind=" + std::to_string(kind) + " (" +
                  aicf::cuda::op_kind_name(static_cast<OpKind>(kind)) + ") status=" +
                  aicf::cuda::status_to_string(st) + " (" + std::to_string(static_cast<int>(st)) + ")";
  if (kernel_id) m += std::string(" kernel_id=") + kernel_id;
  return m;
}

void trace_stderr(const char* what, const char* kernel_id, int kind, const aicf_attr_blob* attr, aicf_stream stream) {
  if (!std::getenv("AICF_TRACE_STDERR")) return;
  if (kernel_id) {
    std::fprintf(stderr, "[aicf][%s] kernel_id=%s kind=%s schema=0x%08x bytes=%u stream=0x%llx\n", what, kernel_id,
                 aicf::cuda::op_kind_name(static_cast<OpKind>(kind)), attr ? attr->schema_id : 0u,
                 attr ? attr->bytes : 0u, static_cast<unsigned long long>(stream));
  } else {
    std::fprintf(stderr, "[aicf][%s] %s (kind=%d) schema=0x%08x bytes=%u stream=0x%llx\n", what,
                 aicf::cuda::op_kind_name(static_cast<OpKind>(kind)), kind, attr ? attr->schema_id : 0u,
                 attr ? attr->bytes : 0u, static_cast<unsigned long long>(stream));
  }
}

// An all-empty blob is passed on as "no attrs", like the reference binding does (bindings.cpp:303-304).
const void* effective_attr(const aicf_attr_blob* a) {
  if (!a) return nullptr;
  if (a->schema_id == 0 && a->bytes == 0 && a->data == nullptr) return nullptr;
  return a;
}

const KernelVariant* lookup(const char* kernel_id, int op_kind) {
  KernelRegistry::ensure_registered();
  return KernelRegistry::instance().find_by_id(static_cast<OpKind>(op_kind), kernel_id);
}

}  // namespace
}  // namespace aicf::capi

using namespace aicf::capi;
using aicf::cuda::OpKind;
using aicf::cuda::Status;

extern "C" {

int aicf_b200_abi_version(void) { return AICF_B200_ABI_VERSION; }
const char* aicf_b200_status_string(int status) { return aicf::cuda::status_to_string(static_cast<Status>(status)); }
const char* aicf_b200_last_error(void) { return t_last_error.c_str(); }
const char* aicf_b200_op_name(int op_kind) { return aicf::cuda::op_kind_name(static_cast<OpKind>(op_kind)); }

int aicf_b200_op_call(int op_kind, const aicf_tensor_desc* inputs, int num_inputs, aicf_tensor_desc* outputs,
                      int num_outputs, const aicf_attr_blob* attr, aicf_stream stream) {
  const Status st = aicf::cuda::dispatch_v0(static_cast<OpKind>(op_kind), as_desc(inputs), num_inputs,
                                            as_desc(outputs), num_outputs, effective_attr(attr), as_stream(stream));
  if (!aicf::cuda::ok(st)) return fail(st, fail_text(op_kind, st, nullptr));
  return AICF_OK;
}

int aicf_b200_launch_by_id(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                           aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr,
                           aicf_stream stream) {
  const Status st =
      aicf::cuda::dispatch_by_id_v0(static_cast<OpKind>(op_kind), kernel_id, as_desc(inputs), num_inputs,
                                    as_desc(outputs), num_outputs, effective_attr(attr), as_stream(stream));
  if (!aicf::cuda::ok(st)) return fail(st, fail_text(op_kind, st, kernel_id ? kernel_id : ""));
  return AICF_OK;
}

int aicf_b200_op_call_traced(int op_kind, const aicf_tensor_desc* inputs, int num_inputs, aicf_tensor_desc* outputs,
                             int num_outputs, const aicf_attr_blob* attr, aicf_stream stream) {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    trace_push_locked(aicf::cuda::op_kind_name(static_cast<OpKind>(op_kind)));
    trace_stderr("op_call", nullptr, op_kind, attr, stream);
  }
  return aicf_b200_op_call(op_kind, inputs, num_inputs, outputs, num_outputs, attr, stream);
}

int aicf_b200_launch_by_id_traced(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                                  aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr,
                                  aicf_stream stream) {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    trace_push_locked(std::string("kid:") + (kernel_id ? kernel_id : "") + " kind:" +
                      aicf::cuda::op_kind_name(static_cast<OpKind>(op_kind)));
    trace_stderr("launch_by_id", kernel_id ? kernel_id : "", op_kind, attr, stream);
  }
  return aicf_b200_launch_by_id(kernel_id, op_kind, inputs, num_inputs, outputs, num_outputs, attr, stream);
}

int aicf_b200_supported(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                        const aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr) {
  const aicf::cuda::KernelVariant* v = lookup(kernel_id, op_kind);
  if (!v || !v->supported) return 0;
  static const aicf::cuda::AttrBlob kEmpty{};
  const aicf::cuda::AttrBlob* a = attr ? as_blob(attr) : &kEmpty;
  if (v->expected_attr_schema_id != 0 && a->schema_id != v->expected_attr_schema_id) return 0;
  return v->supported(as_desc(inputs), num_inputs, as_desc(outputs), num_outputs, a) ? 1 : 0;
}

size_t aicf_b200_query_workspace(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                                 const aicf_attr_blob* attr) {
  const aicf::cuda::KernelVariant* v = lookup(kernel_id, op_kind);
  if (!v || !v->query_workspace) return 0;
  static const aicf::cuda::AttrBlob kEmpty{};
  return v->query_workspace(as_desc(inputs), num_inputs, attr ? as_blob(attr) : &kEmpty);
}

int aicf_b200_launch_ws(const char* kernel_id, int op_kind, const aicf_tensor_desc* inputs, int num_inputs,
                        aicf_tensor_desc* outputs, int num_outputs, const aicf_attr_blob* attr, void* workspace,
                        size_t workspace_bytes, aicf_stream stream) {
  const aicf::cuda::KernelVariant* v = lookup(kernel_id, op_kind);
  if (!v || !v->launch || !v->supported) return fail(Status::NotImplemented, fail_text(op_kind, Status::NotImplemented, kernel_id));
  static const aicf::cuda::AttrBlob kEmpty{};
  const aicf::cuda::AttrBlob* a = attr ? as_blob(attr) : &kEmpty;
  if (v->expected_attr_schema_id != 0 && a->schema_id != v->expected_attr_schema_id)
    return fail(Status::InvalidArgument, fail_text(op_kind, Status::InvalidArgument, kernel_id));
  const Status st = v->launch(as_desc(inputs), num_inputs, as_desc(outputs), num_outputs, a, workspace,
                              workspace_bytes, as_stream(stream));
  if (!aicf::cuda::ok(st)) return fail(st, fail_text(op_kind, st, kernel_id));
  return AICF_OK;
}

int aicf_b200_set_workspace(void* ptr, size_t bytes) {
  aicf::cuda::set_dispatch_workspace(ptr, bytes);
  return AICF_OK;
}

int aicf_b200_num_op_kinds(void) { return static_cast<int>(OpKind::_Count); }

int aicf_b200_kernel_count(int op_kind) {
  aicf::cuda::KernelRegistry::ensure_registered();
  std::vector<const aicf::cuda::KernelVariant*> v;
  aicf::cuda::KernelRegistry::instance().variants_snapshot(static_cast<OpKind>(op_kind), v);
  return static_cast<int>(v.size());
}

const char* aicf_b200_kernel_id(int op_kind, int index) {
  aicf::cuda::KernelRegistry::ensure_registered();
  std::vector<const aicf::cuda::KernelVariant*> v;
  aicf::cuda::KernelRegistry::instance().variants_snapshot(static_cast<OpKind>(op_kind), v);
  if (index < 0 || index >= static_cast<int>(v.size())) return nullptr;
  return v[static_cast<size_t>(index)]->kernel_id;  // string literals: stable for the process lifetime
}

int aicf_b200_gemm_reload_tuning(void) {
  aicf::cuda::gemm_reload_env_overrides();
  return AICF_OK;
}
int aicf_b200_gemm_status(int clear) { return aicf::cuda::gemm_tcgen05_status(clear != 0); }
int aicf_b200_gemm_timeline(int enable, uint64_t* out16) {
  return aicf::cuda::gemm_tcgen05_timeline(enable, reinterpret_cast<unsigned long long*>(out16)) == 0 ? AICF_OK : AICF_INTERNAL;
}
int aicf_b200_wait_status(int clear) {
  const int g = aicf::cuda::gemm_tcgen05_status(clear != 0);
  const int rs = aicf::cuda::row_pipeline_status(clear != 0);
  const int rl = aicf::cuda::layernorm_pipeline_status(clear != 0);
  const int ra = aicf::cuda::adam_pipeline_status(clear != 0);
  const int d = aicf::cuda::dp_wait_status(clear != 0);
  if (g < 0 || rs < 0 || rl < 0 || ra < 0 || d < 0) return -1;
  const int r = rs | rl | ra;
  return (g & 0xFFFF) | (r ? 0x10000 : 0) | ((d & 3) << 17);
}

// ---- trace ------------------------------------------------------------------------------------
void aicf_b200_trace_enable(int flag) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_trace_on = flag != 0;
}
void aicf_b200_trace_reset(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_trace.clear();
}
int aicf_b200_trace_count(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  return static_cast<int>(g_trace.size());
}
const char* aicf_b200_trace_get(int index) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (index < 0 || index >= static_cast<int>(g_trace.size())) return nullptr;
  g_trace_scratch = g_trace[static_cast<size_t>(index)];
  return g_trace_scratch.c_str();
}

// ---- global graph -------------------------------------------------------------------------------
int aicf_b200_graph_begin(aicf_stream* stream_out) {
  std::lock_guard<std::mutex> lock(g_mu);
  std::fprintf(stderr, "[aicf] graph_begin (dedicated stream)\n");
  g_trace.clear();
  g_graph.reset();
  if (!g_graph.stream) {
    const int rc = check_cuda(cudaStreamCreateWithFlags(&g_graph.stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    if (rc != AICF_OK) return rc;
  }
  const int rc = check_cuda(cudaStreamBeginCapture(g_graph.stream, cudaStreamCaptureModeGlobal), "cudaStreamBeginCapture");
  if (rc != AICF_OK) return rc;
  g_graph.capturing = true;
  if (stream_out) *stream_out = from_stream(g_graph.stream);
  return AICF_OK;
}

int aicf_b200_graph_end(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_graph.capturing) return fail(Status::InvalidArgument, "graph_end called but not capturing");
  g_graph.capturing = false;
  int rc = check_cuda(cudaStreamEndCapture(g_graph.stream, &g_graph.graph), "cudaStreamEndCapture");
  if (rc != AICF_OK) {
    g_graph.graph = nullptr;
    return rc;
  }
  rc = check_cuda(cudaGraphInstantiate(&g_graph.exec, g_graph.graph, nullptr, nullptr, 0), "cudaGraphInstantiate");
  if (rc != AICF_OK) {
    g_graph.drop_graph();
    return rc;
  }
  g_graph.captured = true;
  return AICF_OK;
}

int aicf_b200_graph_launch(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_graph.captured || !g_graph.exec) return fail(Status::InvalidArgument, "graph_launch called but no captured graph exists");
  return check_cuda(cudaGraphLaunch(g_graph.exec, g_graph.stream), "cudaGraphLaunch");
}

int aicf_b200_graph_reset(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_graph.reset();
  g_trace.clear();
  return AICF_OK;
}

aicf_stream aicf_b200_graph_stream(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  return from_stream(g_graph.stream);
}

// ---- device helpers -----------------------------------------------------------------------------
int aicf_b200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
int aicf_b200_set_device(int device) { return check_cuda(cudaSetDevice(device), "cudaSetDevice"); }
int aicf_b200_device_info(int device, int64_t* l2_bytes, int* sm_count, int64_t* total_bytes) {
  int l2 = 0, sms = 0;
  if (int rc = check_cuda(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, device), "cudaDeviceGetAttribute(L2)")) return rc;
  if (int rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute(SMs)"))
    return rc;
  if (l2_bytes) *l2_bytes = l2;
  if (sm_count) *sm_count = sms;
  if (total_bytes) {
    cudaDeviceProp prop{};
    if (int rc = check_cuda(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return rc;
    *total_bytes = static_cast<int64_t>(prop.totalGlobalMem);
  }
  return AICF_OK;
}
int aicf_b200_device_pci_bus_id(int device, char* out, int capacity) {
  if (!out || capacity < 13) return fail(Status::InvalidArgument, "device_pci_bus_id: need a buffer of at least 13 bytes");
  return check_cuda(cudaDeviceGetPCIBusId(out, capacity, device), "cudaDeviceGetPCIBusId");
}
int aicf_b200_stream_probe(int reads, int writes, const void* const* inputs, void* const* outputs, size_t bytes_each,
                           int packets_in_flight, int blocks_per_sm, aicf_stream stream) {
  const Status st = aicf::cuda::stream_probe(reads, writes, inputs, outputs, bytes_each, packets_in_flight, blocks_per_sm,
                                             reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream)));
  if (!aicf::cuda::ok(st)) return fail(st, std::string("stream_probe: ") + aicf::cuda::status_to_string(st));
  return AICF_OK;
}
int aicf_b200_malloc(void** ptr, size_t bytes) {
  if (!ptr) return fail(Status::InvalidArgument, "malloc: null out pointer");
  return check_cuda(cudaMalloc(ptr, bytes ? bytes : 1), "cudaMalloc");
}
int aicf_b200_free(void* ptr) { return check_cuda(cudaFree(ptr), "cudaFree"); }
int aicf_b200_host_alloc_pinned(void** ptr, size_t bytes) {
  if (!ptr) return fail(Status::InvalidArgument, "host_alloc_pinned: null out pointer");
  return check_cuda(cudaMallocHost(ptr, bytes ? bytes : 1), "cudaMallocHost");
}
int aicf_b200_host_alloc_staging(void** ptr, size_t bytes) {
  if (!ptr) return fail(Status::InvalidArgument, "host_alloc_staging: null out pointer");
  return check_cuda(cudaHostAlloc(ptr, bytes ? bytes : 1, cudaHostAllocWriteCombined), "cudaHostAlloc(write-combined)");
}
int aicf_b200_host_free_pinned(void* ptr) { return check_cuda(cudaFreeHost(ptr), "cudaFreeHost"); }
int aicf_b200_memcpy_h2d(void* dst, const void* src, size_t bytes, aicf_stream stream) {
  return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)), "cudaMemcpyAsync(h2d)");
}
int aicf_b200_memcpy_d2h(void* dst, const void* src, size_t bytes, aicf_stream stream) {
  return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)), "cudaMemcpyAsync(d2h)");
}
int aicf_b200_memcpy_d2d(void* dst, const void* src, size_t bytes, aicf_stream stream) {
  return check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)), "cudaMemcpyAsync(d2d)");
}
int aicf_b200_memset(void* dst, int value, size_t bytes, aicf_stream stream) {
  return check_cuda(cudaMemsetAsync(dst, value, bytes, as_stream(stream)), "cudaMemsetAsync");
}
int aicf_b200_stream_create(aicf_stream* out) {
  if (!out) return fail(Status::InvalidArgument, "stream_create: null out pointer");
  cudaStream_t s = nullptr;
  const int rc = check_cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
  *out = from_stream(s);
  return rc;
}
int aicf_b200_stream_destroy(aicf_stream s) { return check_cuda(cudaStreamDestroy(as_stream(s)), "cudaStreamDestroy"); }
int aicf_b200_stream_sync(aicf_stream s) { return check_cuda(cudaStreamSynchronize(as_stream(s)), "cudaStreamSynchronize"); }
int aicf_b200_device_sync(void) { return check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"); }
int aicf_b200_event_create(uint64_t* out) {
  if (!out) return fail(Status::InvalidArgument, "event_create: null out pointer");
  cudaEvent_t e = nullptr;
  const int rc = check_cuda(cudaEventCreate(&e), "cudaEventCreate");
  *out = static_cast<uint64_t>(reinterpret_cast<uintptr_t>(e));
  return rc;
}
static cudaEvent_t as_event(uint64_t e) { return reinterpret_cast<cudaEvent_t>(static_cast<uintptr_t>(e)); }
int aicf_b200_event_destroy(uint64_t ev) { return check_cuda(cudaEventDestroy(as_event(ev)), "cudaEventDestroy"); }
int aicf_b200_event_record(uint64_t ev, aicf_stream s) { return check_cuda(cudaEventRecord(as_event(ev), as_stream(s)), "cudaEventRecord"); }
int aicf_b200_event_sync(uint64_t ev) { return check_cuda(cudaEventSynchronize(as_event(ev)), "cudaEventSynchronize"); }
int aicf_b200_event_elapsed_ms(uint64_t start, uint64_t stop, float* ms) {
  if (!ms) return fail(Status::InvalidArgument, "event_elapsed_ms: null out pointer");
  return check_cuda(cudaEventElapsedTime(ms, as_event(start), as_event(stop)), "cudaEventElapsedTime");
}
int aicf_b200_stream_wait_event(aicf_stream s, uint64_t ev) {
  return check_cuda(cudaStreamWaitEvent(as_stream(s), as_event(ev), 0), "cudaStreamWaitEvent");
}

}  // extern "C"
