// Captured execution plan (C++ counterpart of the reference's Python PlannedExecutor).
//
// Built from a lowered-op list; at finalize() every decision that the reference repeats on each
// Python call is taken once: op name -> OpKind, kernel id -> KernelVariant*, tensors -> TensorDesc
// arrays, attrs -> AttrBlob, scratch -> one shared workspace. STATIC values are carved from a single
// arena; two values share bytes when their live ranges (first definition .. last use, in op order)
// do not overlap. The reference allocates one torch tensor per value (core_v2/plan.py:174-209).
//
// all_reduce ops run on a second stream: they wait for the op that produced the gradient, and the
// first later op touching that gradient waits for them, so the exchange overlaps the rest of the
// backward pass both in eager runs and inside the captured graph.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../capi/capi_internal.hpp"
#include "aicf/backends/cuda/nvtx.hpp"

using aicf::cuda::AttrBlob;
using aicf::cuda::DType;
using aicf::cuda::KernelRegistry;
using aicf::cuda::KernelVariant;
using aicf::cuda::OpKind;
using aicf::cuda::Status;
using aicf::cuda::TensorDesc;
using namespace aicf::capi;

namespace aicf::cuda {
size_t dp_control_bytes();
bool dp_register_pool(void* mine, size_t bytes, void* const* peers, int rank, int world);
void dp_unregister_pool(void* mine);
}  // namespace aicf::cuda

namespace {

constexpr size_t kAlign = 256;
size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Lowered-op names (reference: _OPNAME_TO_KIND, python/aicf_fw/core_v2/exec.py:178-201) + additions.
bool kind_of(const std::string& name, OpKind* k) {
  static const std::map<std::string, OpKind> kMap = {
      {"add", OpKind::EltwiseAdd},        {"relu", OpKind::EltwiseRelu},      {"gemm", OpKind::Gemm},
      {"bias_add", OpKind::BiasAdd},      {"reduce_sum", OpKind::ReduceSum},  {"mse_grad", OpKind::MseGrad},
      {"relu_bwd", OpKind::ReluBwd},      {"sgd_step", OpKind::SgdStep},      {"copy", OpKind::Copy},
      {"copy_saved", OpKind::Copy},       {"copy_aux", OpKind::Copy},         {"grad_zero", OpKind::GradZero},
      {"adam_step", OpKind::AdamStep},    {"step_inc", OpKind::StepInc},      {"bias_corr", OpKind::BiasCorr},
      {"layernorm_fwd", OpKind::LayerNormFwd}, {"layernorm_bwd", OpKind::LayerNormBwd},
      {"batchnorm_fwd", OpKind::BatchNormFwd}, {"batchnorm_bwd", OpKind::BatchNormBwd},
      {"gemm_epilogue", OpKind::GemmEpilogue}, {"softmax", OpKind::Softmax}, {"softmax_ce", OpKind::SoftmaxCE},
      {"reduce_max", OpKind::ReduceMax},  {"reduce_mean", OpKind::ReduceMean}, {"all_reduce", OpKind::AllReduce},
      {"cast", OpKind::Cast},             {"gemm_relu_bwd", OpKind::GemmReluBwd},
      {"dp_adam_step", OpKind::DpAdamStep},
  };
  auto it = kMap.find(name);
  if (it == kMap.end()) return false;
  *k = it->second;
  return true;
}

struct Value {
  int vid = -1;
  std::string name;
  DType dtype = DType::kUnknown;
  int rank = 0;
  int64_t shape[4] = {0, 0, 0, 0};
  int role = AICF_ROLE_STATIC;
  bool persistent = false;
  bool zero_init = false;
  int alias_of = -1;
  void* ptr = nullptr;
  bool bound = false;   // caller-owned memory
  bool peer_visible = false;  // lives in the pool that other ranks map (gradients, broadcast working copies)
  size_t bytes = 0;
  int first = -1, last = -1;  // live range in op indices
};

struct Op {
  std::string op_name;
  OpKind kind{};
  std::string kernel_id;
  std::vector<int> in, out;
  uint32_t schema = 0;
  std::string attr;
  const KernelVariant* variant = nullptr;
  std::vector<TensorDesc> in_desc, out_desc;
  AttrBlob blob{};
  size_t ws_bytes = 0;
  cudaEvent_t ev_ready = nullptr, ev_done = nullptr;  // all_reduce only
};

}  // namespace

struct aicf_plan {
  std::string name;
  std::map<int, Value> values;
  std::vector<Op> ops;
  bool finalized = false;
  void* arena = nullptr;
  size_t pooled_bytes = 0;
  size_t arena_bytes = 0, no_reuse_bytes = 0;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  std::vector<void*> owned;
  void* peer_pool = nullptr;       // one allocation: control block + every peer-visible value
  size_t peer_pool_bytes = 0;
  std::vector<void*> peer_mapped;  // other ranks' pools opened through IPC handles
  bool peers_open = false;
  std::vector<void*> peer_bases;   // every rank's pool as seen from this device (own entry = peer_pool)
  int peer_world = 1;
  cudaStream_t stream = nullptr, comm_stream = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int device = 0;

  Value* find(int vid) {
    auto it = values.find(vid);
    return it == values.end() ? nullptr : &it->second;
  }
  Value* resolve(int vid) {  // follows alias links
    Value* v = find(vid);
    for (int hop = 0; v && v->alias_of >= 0 && hop < 64; ++hop) v = find(v->alias_of);
    return v;
  }
  void drop_graph() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    exec = nullptr;
    graph = nullptr;
  }
};

namespace {

TensorDesc desc_of(const Value& v, void* ptr) {
  TensorDesc d{};
  d.data = ptr;
  d.dtype = v.dtype;
  d.r.rank = v.rank;
  int64_t st = 1;
  for (int i = v.rank - 1; i >= 0; --i) {
    d.shape[i] = v.shape[i];
    d.stride[i] = st;
    st *= v.shape[i];
  }
  d.contiguous = true;
  d.alignment = 256;
  return d;
}

// First-fit interval allocator over op order. Returns the arena size; fills offsets.
size_t assign_arena(std::vector<Value*>& vals, int num_ops, std::map<int, size_t>* offsets) {
  struct Block { size_t off, size; };
  std::vector<Block> free_list;
  size_t top = 0;
  std::vector<std::vector<Value*>> starts(static_cast<size_t>(num_ops) + 1), ends(static_cast<size_t>(num_ops) + 1);
  for (Value* v : vals) {
    starts[static_cast<size_t>(v->first)].push_back(v);
    ends[static_cast<size_t>(v->last)].push_back(v);
  }
  for (int i = 0; i < num_ops; ++i) {
    auto& s = starts[static_cast<size_t>(i)];
    std::sort(s.begin(), s.end(), [](const Value* a, const Value* b) { return a->bytes > b->bytes; });
    for (Value* v : s) {
      const size_t need = round_up(v->bytes, kAlign);
      size_t best = free_list.size();
      for (size_t k = 0; k < free_list.size(); ++k)
        if (free_list[k].size >= need && (best == free_list.size() || free_list[k].size < free_list[best].size)) best = k;
      size_t off;
      if (best != free_list.size()) {
        off = free_list[best].off;
        if (free_list[best].size == need) {
          free_list.erase(free_list.begin() + static_cast<std::ptrdiff_t>(best));
        } else {
          free_list[best].off += need;
          free_list[best].size -= need;
        }
      } else if (!free_list.empty() && free_list.back().off + free_list.back().size == top) {
        // grow the trailing free block instead of leaving a hole below the new top
        off = free_list.back().off;
        top = off + need;
        free_list.pop_back();
      } else {
        off = top;
        top += need;
      }
      (*offsets)[v->vid] = off;
    }
    for (Value* v : ends[static_cast<size_t>(i)]) {
      Block b{(*offsets)[v->vid], round_up(v->bytes, kAlign)};
      auto pos = std::lower_bound(free_list.begin(), free_list.end(), b,
                                  [](const Block& x, const Block& y) { return x.off < y.off; });
      pos = free_list.insert(pos, b);
      // coalesce with neighbours
      if (pos + 1 != free_list.end() && pos->off + pos->size == (pos + 1)->off) {
        pos->size += (pos + 1)->size;
        free_list.erase(pos + 1);
      }
      if (pos != free_list.begin() && (pos - 1)->off + (pos - 1)->size == pos->off) {
        (pos - 1)->size += pos->size;
        free_list.erase(pos);
      }
    }
  }
  return top;
}

int enqueue_all(aicf_plan* p, cudaStream_t main, std::vector<cudaEvent_t>* marks = nullptr) {
  // Values in use by ops forked to the communication stream, and the event that ends that use: `pending` holds what
  // a forked op writes (a later reader or writer on `main` waits), `pending_reads` what it only reads (a later
  // WRITER on `main` waits: write after read). The communication stream runs its ops in order, so the event of the
  // latest forked op that touches a value covers the earlier ones.
  std::map<int, cudaEvent_t> pending, pending_reads;
  // AICF_PLAN_NO_OVERLAP=1 keeps the exchange on the main stream (to measure what the side stream buys)
  static const bool no_overlap = std::getenv("AICF_PLAN_NO_OVERLAP") != nullptr;
  const bool overlap = (aicf_b200_dp_world_size() > 1 || p->peer_world > 1) && !marks && !no_overlap;
  for (size_t i = 0; i < p->ops.size(); ++i) {
    Op& op = p->ops[i];
    if (marks)
      if (int rc = check_cuda(cudaEventRecord((*marks)[i], main), "cudaEventRecord(profile)")) return rc;
    auto wait_for = [&](int vid) -> int {
      Value* v = p->resolve(vid);
      if (!v) return AICF_OK;
      auto it = pending.find(v->vid);
      if (it == pending.end()) return AICF_OK;
      const int rc = check_cuda(cudaStreamWaitEvent(main, it->second, 0), "cudaStreamWaitEvent(join)");
      pending.erase(it);
      return rc;
    };
    auto wait_for_readers = [&](int vid) -> int {
      Value* v = p->resolve(vid);
      if (!v) return AICF_OK;
      auto it = pending_reads.find(v->vid);
      if (it == pending_reads.end()) return AICF_OK;
      const int rc = check_cuda(cudaStreamWaitEvent(main, it->second, 0), "cudaStreamWaitEvent(join readers)");
      pending_reads.erase(it);
      return rc;
    };
    for (int vid : op.in)
      if (int rc = wait_for(vid)) return rc;
    for (int vid : op.out) {
      if (int rc = wait_for(vid)) return rc;
      if (int rc = wait_for_readers(vid)) return rc;
    }

    cudaStream_t s = main;
    const bool on_comm = overlap && (op.kind == OpKind::AllReduce || op.kind == OpKind::DpAdamStep) && op.ev_ready && op.ev_done;
    if (on_comm) {
      if (int rc = check_cuda(cudaEventRecord(op.ev_ready, main), "cudaEventRecord(fork)")) return rc;
      if (int rc = check_cuda(cudaStreamWaitEvent(p->comm_stream, op.ev_ready, 0), "cudaStreamWaitEvent(fork)")) return rc;
      s = p->comm_stream;
    }
    AICF_NVTX_RANGE(op.variant->kernel_id);  // eager: the launch; under capture: the recording of the op's node
    const Status st = op.variant->launch(op.in_desc.data(), static_cast<int>(op.in_desc.size()), op.out_desc.data(),
                                         static_cast<int>(op.out_desc.size()), &op.blob, op.ws_bytes ? p->ws : nullptr,
                                         op.ws_bytes ? p->ws_bytes : 0, s);
    if (!aicf::cuda::ok(st)) {
      return fail(st, "[plan " + p->name + "] op #" + std::to_string(i) + " '" + op.op_name + "' kernel_id=" +
                          (op.variant->kernel_id ? op.variant->kernel_id : "?") + " failed: " +
                          aicf::cuda::status_to_string(st));
    }
    if (on_comm) {
      if (int rc = check_cuda(cudaEventRecord(op.ev_done, p->comm_stream), "cudaEventRecord(done)")) return rc;
      for (int vid : op.out) {
        Value* v = p->resolve(vid);
        if (v) pending[v->vid] = op.ev_done;
      }
      for (int vid : op.in) {
        Value* v = p->resolve(vid);
        if (v && !pending.count(v->vid)) pending_reads[v->vid] = op.ev_done;
      }
    }
  }
  for (auto& kv : pending)  // every forked branch rejoins before the step ends
    if (int rc = check_cuda(cudaStreamWaitEvent(main, kv.second, 0), "cudaStreamWaitEvent(final join)")) return rc;
  for (auto& kv : pending_reads)
    if (int rc = check_cuda(cudaStreamWaitEvent(main, kv.second, 0), "cudaStreamWaitEvent(final join)")) return rc;
  if (marks)
    if (int rc = check_cuda(cudaEventRecord(marks->back(), main), "cudaEventRecord(profile)")) return rc;
  return AICF_OK;
}

}  // namespace

extern "C" {

aicf_plan* aicf_b200_plan_create(const char* name) {
  aicf_plan* p = new aicf_plan();
  p->name = name ? name : "plan";
  return p;
}

void aicf_b200_plan_destroy(aicf_plan* p) {
  if (!p) return;
  if (p->stream) cudaStreamSynchronize(p->stream);
  if (p->comm_stream) cudaStreamSynchronize(p->comm_stream);
  p->drop_graph();
  for (Op& op : p->ops) {
    if (op.ev_ready) cudaEventDestroy(op.ev_ready);
    if (op.ev_done) cudaEventDestroy(op.ev_done);
  }
  for (void* q : p->owned) cudaFree(q);
  if (p->peer_pool) {
    aicf::cuda::dp_unregister_pool(p->peer_pool);
    for (void* q : p->peer_mapped)
      if (q) cudaIpcCloseMemHandle(q);
    cudaFree(p->peer_pool);
  }
  if (p->arena) cudaFree(p->arena);
  if (p->ws) cudaFree(p->ws);
  if (p->stream) cudaStreamDestroy(p->stream);
  if (p->comm_stream) cudaStreamDestroy(p->comm_stream);
  cudaGetLastError();
  delete p;
}

int aicf_b200_plan_add_value(aicf_plan* p, int vid, const char* name, int dtype, int rank, const int64_t* shape,
                             int role, int persistent, int zero_init) {
  if (!p || p->finalized) return fail(Status::InvalidArgument, "plan_add_value: plan missing or finalized");
  if (rank < 0 || rank > aicf::cuda::kMaxRank || (rank > 0 && !shape))
    return fail(Status::InvalidArgument, "plan_add_value: bad rank/shape");
  if (role < AICF_ROLE_INPUT || role > AICF_ROLE_STATIC) return fail(Status::InvalidArgument, "plan_add_value: bad role");
  const DType dt = static_cast<DType>(dtype);
  if (aicf::cuda::dtype_size_bytes(dt) == 0) return fail(Status::InvalidArgument, "plan_add_value: bad dtype");
  if (p->values.count(vid)) return fail(Status::InvalidArgument, "plan_add_value: duplicate value id");
  Value v;
  v.vid = vid;
  v.name = name ? name : "";
  v.dtype = dt;
  v.rank = rank;
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) {
    if (shape[i] <= 0) return fail(Status::InvalidArgument, "plan_add_value: non-positive extent");
    v.shape[i] = shape[i];
    n *= shape[i];
  }
  v.bytes = static_cast<size_t>(n) * static_cast<size_t>(aicf::cuda::dtype_size_bytes(dt));
  v.role = role;
  v.persistent = persistent != 0 || role != AICF_ROLE_STATIC;
  v.zero_init = zero_init != 0;
  p->values.emplace(vid, v);
  return AICF_OK;
}

int aicf_b200_plan_add_op(aicf_plan* p, const char* op_name, const char* kernel_id, const int* inputs, int num_inputs,
                          const int* outputs, int num_outputs, uint32_t schema_id, const void* attr_bytes,
                          uint32_t attr_len) {
  if (!p || p->finalized || !op_name) return fail(Status::InvalidArgument, "plan_add_op: plan missing or finalized");
  if (num_inputs < 0 || num_outputs < 0 || (num_inputs && !inputs) || (num_outputs && !outputs))
    return fail(Status::InvalidArgument, "plan_add_op: bad operand lists");
  Op op;
  op.op_name = op_name;
  if (!kind_of(op.op_name, &op.kind))
    return fail(Status::InvalidArgument, std::string("[exec] unsupported lowered op '") + op_name + "' (no OpKind mapping)");
  if (kernel_id && kernel_id[0]) op.kernel_id = kernel_id;
  op.in.assign(inputs, inputs + num_inputs);
  op.out.assign(outputs, outputs + num_outputs);
  for (int vid : op.in)
    if (!p->find(vid)) return fail(Status::InvalidArgument, "plan_add_op: unknown input value id " + std::to_string(vid));
  for (int vid : op.out)
    if (!p->find(vid)) return fail(Status::InvalidArgument, "plan_add_op: unknown output value id " + std::to_string(vid));
  op.schema = schema_id;
  if (attr_bytes && attr_len) op.attr.assign(static_cast<const char*>(attr_bytes), attr_len);
  p->ops.push_back(std::move(op));
  return AICF_OK;
}

int aicf_b200_plan_alias(aicf_plan* p, int vid, int target_vid) {
  if (!p || p->finalized) return fail(Status::InvalidArgument, "plan_alias: plan missing or finalized");
  Value* v = p->find(vid);
  Value* t = p->resolve(target_vid);
  if (!v || !t || t->vid == vid) return fail(Status::InvalidArgument, "plan_alias: unknown value id");
  if (v->bytes != t->bytes || v->dtype != t->dtype) return fail(Status::InvalidArgument, "plan_alias: size/dtype mismatch");
  v->alias_of = t->vid;
  return AICF_OK;
}

int aicf_b200_plan_bind(aicf_plan* p, int vid, void* device_ptr) {
  if (!p || p->finalized || !device_ptr) return fail(Status::InvalidArgument, "plan_bind: plan missing/finalized or null pointer");
  Value* v = p->find(vid);
  if (!v || v->alias_of >= 0) return fail(Status::InvalidArgument, "plan_bind: unknown or aliased value id");
  v->ptr = device_ptr;
  v->bound = true;
  return AICF_OK;
}

int aicf_b200_plan_set_peer_visible(aicf_plan* p, int vid) {
  if (!p || p->finalized) return fail(Status::InvalidArgument, "plan_set_peer_visible: plan missing or finalized");
  Value* v = p->find(vid);
  if (!v) return fail(Status::InvalidArgument, "plan_set_peer_visible: unknown value id");
  v->peer_visible = true;
  v->persistent = true;
  return AICF_OK;
}

int aicf_b200_plan_peer_handle(aicf_plan* p, void* handle64, size_t* pool_bytes) {
  if (!p || !p->finalized || !handle64) return fail(Status::InvalidArgument, "plan_peer_handle: plan not finalized or null output");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size is part of the ABI");
  if (pool_bytes) *pool_bytes = p->peer_pool_bytes;
  std::memset(handle64, 0, 64);
  if (!p->peer_pool) return AICF_OK;  // nothing to share
  cudaIpcMemHandle_t h;
  if (int rc = check_cuda(cudaIpcGetMemHandle(&h, p->peer_pool), "cudaIpcGetMemHandle")) return rc;
  std::memcpy(handle64, &h, 64);
  return AICF_OK;
}

int aicf_b200_plan_open_peers(aicf_plan* p, int rank, int world, const void* handles) {
  if (!p || !p->finalized) return fail(Status::InvalidArgument, "plan_open_peers: plan not finalized");
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(Status::InvalidArgument, "plan_open_peers: bad rank/world");
  if (!p->peer_pool) return AICF_OK;
  if (p->peers_open) return fail(Status::InvalidArgument, "plan_open_peers: already open");
  if (world > 1 && !handles) return fail(Status::InvalidArgument, "plan_open_peers: null handles");
  std::vector<void*> bases(static_cast<size_t>(world), nullptr);
  p->peer_mapped.assign(static_cast<size_t>(world), nullptr);
  for (int k = 0; k < world; ++k) {
    if (k == rank) {
      bases[static_cast<size_t>(k)] = p->peer_pool;
      continue;
    }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const uint8_t*>(handles) + 64 * static_cast<size_t>(k), 64);
    void* q = nullptr;
    if (int rc = check_cuda(cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return rc;
    p->peer_mapped[static_cast<size_t>(k)] = q;
    bases[static_cast<size_t>(k)] = q;
  }
  if (!aicf::cuda::dp_register_pool(p->peer_pool, p->peer_pool_bytes, bases.data(), rank, world))
    return fail(Status::Internal, "plan_open_peers: pool registration failed");
  p->peers_open = true;
  p->peer_world = world;
  p->peer_bases = bases;
  return AICF_OK;
}

int aicf_b200_plan_open_peers_raw(aicf_plan* p, int rank, int world, void* const* bases) {
  if (!p || !p->finalized) return fail(Status::InvalidArgument, "plan_open_peers_raw: plan not finalized");
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !bases) return fail(Status::InvalidArgument, "plan_open_peers_raw: bad arguments");
  if (!p->peer_pool) return AICF_OK;
  if (p->peers_open) return fail(Status::InvalidArgument, "plan_open_peers_raw: already open");
  std::vector<void*> b(bases, bases + world);
  b[static_cast<size_t>(rank)] = p->peer_pool;
  for (void* q : b)
    if (!q) return fail(Status::InvalidArgument, "plan_open_peers_raw: null pool address");
  if (!aicf::cuda::dp_register_pool(p->peer_pool, p->peer_pool_bytes, b.data(), rank, world))
    return fail(Status::Internal, "plan_open_peers_raw: pool registration failed");
  p->peers_open = true;
  p->peer_world = world;
  p->peer_bases = b;
  return AICF_OK;
}

int aicf_b200_plan_finalize(aicf_plan* p) {
  if (!p || p->finalized) return fail(Status::InvalidArgument, "plan_finalize: plan missing or already finalized");
  KernelRegistry::ensure_registered();
  cudaGetDevice(&p->device);
  const int nops = static_cast<int>(p->ops.size());

  // live ranges on alias-resolved values
  for (int i = 0; i < nops; ++i) {
    for (const std::vector<int>* lst : {&p->ops[static_cast<size_t>(i)].in, &p->ops[static_cast<size_t>(i)].out})
      for (int vid : *lst) {
        Value* v = p->resolve(vid);
        if (!v) return fail(Status::InvalidArgument, "plan_finalize: dangling alias");
        if (v->first < 0) v->first = i;
        v->last = i;
      }
  }
  // Ops that may run on the communication stream (all_reduce, dp_adam_step) finish at an unknown point after their
  // position in op order, so every value they touch stays live to the end of the step: its arena bytes are never
  // handed to a value that a later main-stream op writes while the exchange may still be reading.
  for (int i = 0; i < nops; ++i) {
    const Op& op = p->ops[static_cast<size_t>(i)];
    if (op.kind != OpKind::AllReduce && op.kind != OpKind::DpAdamStep) continue;
    for (const std::vector<int>* lst : {&op.in, &op.out})
      for (int vid : *lst)
        if (Value* v = p->resolve(vid)) v->last = nops - 1;
  }
  // a value that is an alias target of a persistent value is persistent too
  for (auto& kv : p->values)
    if (kv.second.alias_of >= 0 && kv.second.persistent) {
      Value* t = p->resolve(kv.first);
      if (t) t->persistent = true;
    }

  // peer-visible values: one pool that starts with the exchange's control block
  {
    size_t pool = aicf::cuda::dp_control_bytes();
    bool any = false;
    for (auto& kv : p->values) {
      Value& v = kv.second;
      if (v.alias_of >= 0 || v.bound || !v.peer_visible) continue;
      any = true;
      pool += round_up(v.bytes, kAlign);
    }
    if (any) {
      if (int rc = check_cuda(cudaMalloc(&p->peer_pool, pool), "cudaMalloc(peer pool)")) return rc;
      if (int rc = check_cuda(cudaMemset(p->peer_pool, 0, pool), "cudaMemset(peer pool)")) return rc;
      p->peer_pool_bytes = pool;
      size_t off = aicf::cuda::dp_control_bytes();
      for (auto& kv : p->values) {
        Value& v = kv.second;
        if (v.alias_of >= 0 || v.bound || !v.peer_visible) continue;
        v.ptr = static_cast<uint8_t*>(p->peer_pool) + off;
        off += round_up(v.bytes, kAlign);
      }
    }
  }

  std::vector<Value*> arena_vals;
  p->no_reuse_bytes = 0;
  for (auto& kv : p->values) {
    Value& v = kv.second;
    if (v.alias_of >= 0 || v.bound) continue;
    if (v.peer_visible && v.ptr) {
      if (v.role == AICF_ROLE_STATIC) p->no_reuse_bytes += round_up(v.bytes, kAlign);
      continue;
    }
    if (v.role == AICF_ROLE_STATIC) p->no_reuse_bytes += round_up(v.bytes, kAlign);
    if (v.role == AICF_ROLE_STATIC && !v.persistent && !v.zero_init && v.first >= 0) {
      arena_vals.push_back(&v);
    } else {
      void* q = nullptr;
      if (int rc = check_cuda(cudaMalloc(&q, v.bytes ? v.bytes : 1), "cudaMalloc(plan value)")) return rc;
      p->owned.push_back(q);
      v.ptr = q;
      if (v.zero_init || v.role == AICF_ROLE_STATIC)
        if (int rc = check_cuda(cudaMemset(q, 0, v.bytes), "cudaMemset(plan value)")) return rc;
    }
  }
  std::map<int, size_t> offsets;
  p->arena_bytes = assign_arena(arena_vals, nops, &offsets);
  if (p->arena_bytes) {
    if (int rc = check_cuda(cudaMalloc(&p->arena, p->arena_bytes), "cudaMalloc(plan arena)")) return rc;
    if (int rc = check_cuda(cudaMemset(p->arena, 0, p->arena_bytes), "cudaMemset(plan arena)")) return rc;
    for (Value* v : arena_vals) v->ptr = static_cast<uint8_t*>(p->arena) + offsets[v->vid];
  }
  size_t owned_static = 0;
  for (auto& kv : p->values) {
    const Value& v = kv.second;
    if (v.alias_of < 0 && !v.bound && v.role == AICF_ROLE_STATIC &&
        std::find(arena_vals.begin(), arena_vals.end(), &v) == arena_vals.end())
      owned_static += round_up(v.bytes, kAlign);
  }
  p->pooled_bytes = p->arena_bytes;  // extent of the shared arena itself
  p->arena_bytes += owned_static;    // reported figure covers every STATIC byte, pooled or not

  // resolve variants, descriptors, workspace
  size_t ws_need = 0;
  bool any_allreduce = false;
  for (int i = 0; i < nops; ++i) {
    Op& op = p->ops[static_cast<size_t>(i)];
    for (int vid : op.in) {
      Value* v = p->resolve(vid);
      op.in_desc.push_back(desc_of(*p->find(vid), v->ptr));
    }
    for (int vid : op.out) {
      Value* v = p->resolve(vid);
      op.out_desc.push_back(desc_of(*p->find(vid), v->ptr));
    }
    op.blob.schema_id = op.schema;
    op.blob.bytes = static_cast<uint32_t>(op.attr.size());
    op.blob.data = op.attr.empty() ? nullptr : op.attr.data();

    const int ni = static_cast<int>(op.in_desc.size()), no = static_cast<int>(op.out_desc.size());
    const std::string where = "[plan " + p->name + "] op #" + std::to_string(i) + " '" + op.op_name + "'";
    if (!op.kernel_id.empty()) {
      const KernelVariant* v = KernelRegistry::instance().find_by_id(op.kind, op.kernel_id.c_str());
      if (!v) return fail(Status::NotImplemented, where + ": unknown kernel_id " + op.kernel_id);
      if (v->expected_attr_schema_id != 0 && op.blob.schema_id != v->expected_attr_schema_id)
        return fail(Status::InvalidArgument, where + ": attr schema mismatch for " + op.kernel_id);
      if (!v->supported(op.in_desc.data(), ni, op.out_desc.data(), no, &op.blob))
        return fail(Status::InvalidArgument, where + ": kernel " + op.kernel_id + " does not support these operands");
      op.variant = v;
    } else {
      std::vector<const KernelVariant*> vars;
      KernelRegistry::instance().variants_snapshot(op.kind, vars);
      for (const KernelVariant* v : vars) {
        if (!v->supported || !v->launch) continue;
        if (v->expected_attr_schema_id != 0 && op.blob.schema_id != v->expected_attr_schema_id) continue;
        if (v->supported(op.in_desc.data(), ni, op.out_desc.data(), no, &op.blob)) {
          op.variant = v;
          break;
        }
      }
      if (!op.variant) return fail(Status::NotImplemented, where + ": no kernel variant supports these operands");
    }
    if (op.variant->query_workspace) op.ws_bytes = op.variant->query_workspace(op.in_desc.data(), ni, &op.blob);
    ws_need = std::max(ws_need, op.ws_bytes);
    if (op.kind == OpKind::AllReduce || op.kind == OpKind::DpAdamStep) any_allreduce = true;
  }
  if (ws_need) {
    p->ws_bytes = round_up(ws_need, kAlign);
    if (int rc = check_cuda(cudaMalloc(&p->ws, p->ws_bytes), "cudaMalloc(plan workspace)")) return rc;
  }
  if (int rc = check_cuda(cudaStreamCreateWithFlags(&p->stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags")) return rc;
  if (any_allreduce) {
    if (int rc = check_cuda(cudaStreamCreateWithFlags(&p->comm_stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags")) return rc;
    for (Op& op : p->ops)
      if (op.kind == OpKind::AllReduce || op.kind == OpKind::DpAdamStep) {
        if (int rc = check_cuda(cudaEventCreateWithFlags(&op.ev_ready, cudaEventDisableTiming), "cudaEventCreate")) return rc;
        if (int rc = check_cuda(cudaEventCreateWithFlags(&op.ev_done, cudaEventDisableTiming), "cudaEventCreate")) return rc;
      }
  }
  if (int rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize(plan finalize)")) return rc;
  p->finalized = true;
  return AICF_OK;
}

void* aicf_b200_plan_value_ptr(aicf_plan* p, int vid) {
  Value* v = p ? p->resolve(vid) : nullptr;
  return v ? v->ptr : nullptr;
}
size_t aicf_b200_plan_value_bytes(aicf_plan* p, int vid) {
  Value* v = p ? p->find(vid) : nullptr;
  return v ? v->bytes : 0;
}
int64_t aicf_b200_plan_value_arena_offset(aicf_plan* p, int vid) {
  Value* v = p ? p->resolve(vid) : nullptr;
  if (!v || !v->ptr || !p->arena || p->pooled_bytes == 0) return -1;
  const uint8_t* base = static_cast<const uint8_t*>(p->arena);
  const uint8_t* q = static_cast<const uint8_t*>(v->ptr);
  return (q >= base && q < base + p->pooled_bytes) ? static_cast<int64_t>(q - base) : -1;
}
size_t aicf_b200_plan_peer_pool_bytes(aicf_plan* p) { return p ? p->peer_pool_bytes : 0; }
void* aicf_b200_plan_peer_pool_base(aicf_plan* p, int rank) {
  if (!p || rank < 0) return nullptr;
  if (!p->peers_open) return rank == 0 ? p->peer_pool : nullptr;
  return static_cast<size_t>(rank) < p->peer_bases.size() ? p->peer_bases[static_cast<size_t>(rank)] : nullptr;
}
size_t aicf_b200_plan_arena_bytes(aicf_plan* p) { return p ? p->arena_bytes : 0; }
size_t aicf_b200_plan_arena_bytes_no_reuse(aicf_plan* p) { return p ? p->no_reuse_bytes : 0; }
int aicf_b200_plan_num_ops(aicf_plan* p) { return p ? static_cast<int>(p->ops.size()) : 0; }
const char* aicf_b200_plan_op_kernel_id(aicf_plan* p, int i) {
  if (!p || !p->finalized || i < 0 || i >= static_cast<int>(p->ops.size())) return nullptr;
  return p->ops[static_cast<size_t>(i)].variant->kernel_id;
}

int aicf_b200_plan_run(aicf_plan* p, aicf_stream stream) {
  if (!p || !p->finalized) return fail(Status::InvalidArgument, "plan_run: plan not finalized");
  return enqueue_all(p, stream ? as_stream(stream) : p->stream);
}

int aicf_b200_plan_capture(aicf_plan* p) {
  if (!p || !p->finalized) return fail(Status::InvalidArgument, "plan_capture: plan not finalized");
  p->drop_graph();
  if (int rc = check_cuda(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture")) return rc;
  const int rc_ops = enqueue_all(p, p->stream);
  cudaGraph_t g = nullptr;
  const cudaError_t e = cudaStreamEndCapture(p->stream, &g);
  if (rc_ops != AICF_OK) {
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    return rc_ops;
  }
  if (int rc = check_cuda(e, "cudaStreamEndCapture")) return rc;
  p->graph = g;
  if (int rc = check_cuda(cudaGraphInstantiate(&p->exec, p->graph, nullptr, nullptr, 0), "cudaGraphInstantiate")) {
    p->drop_graph();
    return rc;
  }
  return AICF_OK;
}

int aicf_b200_plan_replay(aicf_plan* p, int n) {
  if (!p || !p->exec) return fail(Status::InvalidArgument, "[exec] replay called before capture()");
  for (int i = 0; i < n; ++i)
    if (int rc = check_cuda(cudaGraphLaunch(p->exec, p->stream), "cudaGraphLaunch")) return rc;
  return AICF_OK;
}

int aicf_b200_plan_replay_on(aicf_plan* p, int n, aicf_stream stream) {
  if (!p || !p->exec) return fail(Status::InvalidArgument, "[exec] replay called before capture()");
  cudaStream_t s = stream ? as_stream(stream) : p->stream;
  for (int i = 0; i < n; ++i)
    if (int rc = check_cuda(cudaGraphLaunch(p->exec, s), "cudaGraphLaunch")) return rc;
  return AICF_OK;
}

int aicf_b200_plan_reset_graph(aicf_plan* p) {
  if (!p) return fail(Status::InvalidArgument, "plan_reset_graph: null plan");
  if (p->stream) cudaStreamSynchronize(p->stream);
  p->drop_graph();
  return AICF_OK;
}

aicf_stream aicf_b200_plan_stream(aicf_plan* p) { return p ? from_stream(p->stream) : 0; }

int aicf_b200_plan_sync(aicf_plan* p) {
  if (!p || !p->stream) return fail(Status::InvalidArgument, "plan_sync: plan not finalized");
  if (p->comm_stream)
    if (int rc = check_cuda(cudaStreamSynchronize(p->comm_stream), "cudaStreamSynchronize(comm)")) return rc;
  return check_cuda(cudaStreamSynchronize(p->stream), "cudaStreamSynchronize");
}

int aicf_b200_plan_graph_nodes(aicf_plan* p) {
  if (!p || !p->graph) return -1;
  size_t n = 0;
  if (cudaGraphGetNodes(p->graph, nullptr, &n) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return static_cast<int>(n);
}

int aicf_b200_plan_graph_kernel_nodes(aicf_plan* p) {
  if (!p || !p->graph) return -1;
  size_t n = 0;
  if (cudaGraphGetNodes(p->graph, nullptr, &n) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  std::vector<cudaGraphNode_t> nodes(n);
  if (n && cudaGraphGetNodes(p->graph, nodes.data(), &n) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  int kernels = 0;
  for (cudaGraphNode_t nd : nodes) {
    cudaGraphNodeType t;
    if (cudaGraphNodeGetType(nd, &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
  }
  return kernels;
}

int aicf_b200_plan_profile(aicf_plan* p, float* ms_per_op, int capacity) {
  if (!p || !p->finalized || !ms_per_op) return fail(Status::InvalidArgument, "plan_profile: plan not finalized or null output");
  const size_t n = p->ops.size();
  if (capacity < static_cast<int>(n)) return fail(Status::InvalidArgument, "plan_profile: output too small");
  std::vector<cudaEvent_t> marks(n + 1, nullptr);
  int rc = AICF_OK;
  for (auto& e : marks)
    if (rc == AICF_OK) rc = check_cuda(cudaEventCreate(&e), "cudaEventCreate(profile)");
  if (rc == AICF_OK) rc = enqueue_all(p, p->stream, &marks);
  if (rc == AICF_OK) rc = check_cuda(cudaStreamSynchronize(p->stream), "cudaStreamSynchronize(profile)");
  for (size_t i = 0; i < n && rc == AICF_OK; ++i)
    rc = check_cuda(cudaEventElapsedTime(&ms_per_op[i], marks[i], marks[i + 1]), "cudaEventElapsedTime(profile)");
  for (auto& e : marks)
    if (e) cudaEventDestroy(e);
  return rc;
}

}  // extern "C"
