// Data-parallel optimizer step fused with its gradient exchange, over NVLink peer memory.
//
// One launch per parameter tensor and rank does what all_reduce + adam_step + weight broadcast would do:
//   1. tells every peer "my gradient of this tensor is final and nobody here reads the old weights any more"
//      and waits for the same word from all of them (flags in peer-visible memory, sequence numbers, no reset);
//   2. for ITS shard of the tensor (elements [n*r/N, n*(r+1)/N), 4-aligned): sums the N shard gradients straight
//      out of the peers' gradient buffers (P2P loads, always in rank order 0..N-1, so the sum is bit-reproducible),
//      applies Adam to its shard of the fp32 master weights and moments, and stores the new weights into every
//      rank's working copy (bf16 / f16 copy for matrices, the fp32 parameter itself for biases) with P2P stores;
//   3. tells every peer "my stores into your memory are done" and the last CTA waits for all peers, so kernel
//      completion means this rank's working copies are complete and its gradient buffer may be overwritten.
// Reduce-scatter, update and all-gather travel over NVLink once each (4 B/param in, 2 B/param out per rank for
// matrices) and Adam's 28 B/param of HBM traffic shrinks to 1/N per rank. The kernel uses no shared memory and 64
// registers, so its CTAs co-reside with the persistent GEMM CTAs of the backward pass instead of waiting for SMs.
//
// fp32 master weights and moments of matrices are therefore sharded: rank r's copy is current only inside its
// shard (gather the shards to read a whole master tensor). Working copies and biases are complete on every rank.
//
// Waits are bounded (~2 s); a wait that expires sets a status word, skips the work that depended on it and lets
// the kernel finish. No TMA multicast, no multimem: plain peer loads and stores.
#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "../capi/capi_internal.hpp"
#include "adam_math.cuh"

namespace aicf::cuda {

constexpr int kMaxRanks = 8;
constexpr int kMaxSlots = 60;  // dp_adam_step ops per plan
// Layout of the control block at the start of every peer pool (8 KiB):
//   uint32 flags[kMaxSlots][2][kMaxRanks]   written by peers (phase 0 = ready, phase 1 = done)
//   uint32 epoch[kMaxSlots]; uint32 done[kMaxSlots]   local
constexpr size_t kFlagsBytes = size_t(kMaxSlots) * 2 * kMaxRanks * 4;
constexpr size_t kControlBytes = 8192;
static_assert(kFlagsBytes + size_t(kMaxSlots) * 8 <= kControlBytes, "control block layout");

namespace {

struct PeerPool {
  uint8_t* mine = nullptr;
  size_t bytes = 0;
  uint8_t* peer[kMaxRanks] = {nullptr};
  int rank = 0, world = 1;
};
std::mutex g_pools_mu;
std::vector<PeerPool> g_pools;

const PeerPool* pool_of(const void* p, size_t len) {
  const uint8_t* q = static_cast<const uint8_t*>(p);
  for (const PeerPool& pp : g_pools)
    if (q >= pp.mine + kControlBytes && q + len <= pp.mine + pp.bytes) return &pp;
  return nullptr;
}

__device__ int g_dp_status = 0;  // non-zero: a cross-GPU wait expired (1 = ready phase, 2 = done phase)
constexpr unsigned long long kPeerWaitBudgetNs = 2000000000ull;

struct DpAdamArgs {
  const float* g_of[kMaxRanks];   // gradient buffer of every rank (own included)
  void* bcast_to[kMaxRanks];      // where the new weights go on every rank (own included)
  uint32_t* flags_of[kMaxRanks];  // this op's flag block [2][kMaxRanks] in every rank's pool
  float *p, *m, *v;
  const int32_t* step;
  uint32_t *epoch, *done;
  int64_t begin, end;  // this rank's shard
  int rank, world;
  int bcast_kind;  // 1 bf16, 2 f16, 3 fp32 (the parameter itself)
  AdamHyper h;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until every rank's word in `mine[0..world)` has reached `epoch` (sequence numbers only grow; the
// comparison is wrap-safe). One thread calls it. false = budget exhausted.
__device__ bool wait_all_ranks(const uint32_t* mine, int world, uint32_t epoch) {
  const unsigned long long t0 = now_ns();
  for (int k = 0; k < world; ++k) {
    uint32_t spin = 0;
    while (static_cast<int32_t>(ld_acquire_sys(mine + k) - epoch) < 0) {
      if ((++spin & 63u) == 0u && now_ns() - t0 > kPeerWaitBudgetNs) return false;
    }
  }
  return true;
}

template <int kBcast>
__device__ __forceinline__ void bcast_x4(const DpAdamArgs& a, int64_t packet, const Pack16<float>& po) {
  if (kBcast == 3) {
    const float4 w = make_float4(po.v[0], po.v[1], po.v[2], po.v[3]);
    for (int k = 0; k < a.world; ++k) __stcg(reinterpret_cast<float4*>(a.bcast_to[k]) + packet, w);
  } else {
    uint2 w;
    if (kBcast == 1) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(po.v[0], po.v[1]), hi = __floats2bfloat162_rn(po.v[2], po.v[3]);
      w.x = *reinterpret_cast<const uint32_t*>(&lo);
      w.y = *reinterpret_cast<const uint32_t*>(&hi);
    } else {
      const __half2 lo = __floats2half2_rn(po.v[0], po.v[1]), hi = __floats2half2_rn(po.v[2], po.v[3]);
      w.x = *reinterpret_cast<const uint32_t*>(&lo);
      w.y = *reinterpret_cast<const uint32_t*>(&hi);
    }
    for (int k = 0; k < a.world; ++k) __stcg(reinterpret_cast<uint2*>(a.bcast_to[k]) + packet, w);
  }
}
template <int kBcast>
__device__ __forceinline__ void bcast_x1(const DpAdamArgs& a, int64_t i, float v) {
  for (int k = 0; k < a.world; ++k) {
    if (kBcast == 1) static_cast<__nv_bfloat16*>(a.bcast_to[k])[i] = __float2bfloat16_rn(v);
    if (kBcast == 2) static_cast<__half*>(a.bcast_to[k])[i] = __float2half_rn(v);
    if (kBcast == 3) static_cast<float*>(a.bcast_to[k])[i] = v;
  }
}

template <int kBcast>
__global__ void __launch_bounds__(256) dp_adam_kernel(const DpAdamArgs a) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_go;
  if (threadIdx.x == 0) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;
    s_epoch = e;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int k = 0; k < a.world; ++k) st_release_sys(a.flags_of[k] + 0 * kMaxRanks + a.rank, e);
    }
    const bool ok = wait_all_ranks(a.flags_of[a.rank] + 0 * kMaxRanks, a.world, e);
    if (!ok) atomicCAS(&g_dp_status, 0, 1);
    s_go = ok ? 1 : 0;
  }
  __syncthreads();

  if (s_go) {
    int t = a.step[0];
    if (t < 1) t = 1;
    const float d1 = static_cast<float>(1.0 - pow(static_cast<double>(a.h.beta1), static_cast<double>(t)));
    const float d2 = static_cast<float>(1.0 - pow(static_cast<double>(a.h.beta2), static_cast<double>(t)));
    using V4 = Pack16<float>;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // shard bounds are multiples of 4 except possibly the very end of the tensor
    const int64_t p_begin = a.begin >> 2, p_end = a.end >> 2;
    for (int64_t i = p_begin + tid; i < p_end; i += stride) {
      // all ranks' packets are requested before any is used: up to 8 independent NVLink loads in flight per thread
      float4 gk[kMaxRanks];
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < a.world) gk[k] = __ldcg(reinterpret_cast<const float4*>(a.g_of[k]) + i);
      float4 acc = gk[0];
#pragma unroll
      for (int k = 1; k < kMaxRanks; ++k)  // fixed rank order: the same bits whoever owns the shard
        if (k < a.world) {
          acc.x += gk[k].x;
          acc.y += gk[k].y;
          acc.z += gk[k].z;
          acc.w += gk[k].w;
        }
      const V4 p = ld_stream(reinterpret_cast<const V4*>(a.p) + i);
      const V4 m = ld_stream(reinterpret_cast<const V4*>(a.m) + i);
      const V4 v = ld_stream(reinterpret_cast<const V4*>(a.v) + i);
      const float g[4] = {acc.x, acc.y, acc.z, acc.w};
      V4 po, mo, vo;
#pragma unroll
      for (int e = 0; e < 4; ++e) adam_one<false>(p.v[e], g[e], m.v[e], v.v[e], a.h, d1, d2, po.v[e], mo.v[e], vo.v[e]);
      st_stream(reinterpret_cast<V4*>(a.m) + i, mo);
      st_stream(reinterpret_cast<V4*>(a.v) + i, vo);
      if (kBcast != 3) st_stream(reinterpret_cast<V4*>(a.p) + i, po);
      bcast_x4<kBcast>(a, i, po);
    }
    for (int64_t i = (p_end << 2) + tid; i < a.end; i += stride) {  // ragged end of the last shard
      float g = __ldcg(a.g_of[0] + i);
      for (int k = 1; k < a.world; ++k) g += __ldcg(a.g_of[k] + i);
      float po, mo, vo;
      adam_one<false>(a.p[i], g, a.m[i], a.v[i], a.h, d1, d2, po, mo, vo);
      a.m[i] = mo;
      a.v[i] = vo;
      if (kBcast != 3) a.p[i] = po;
      bcast_x1<kBcast>(a, i, po);
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // this CTA's peer stores are ordered before its arrival below
    const unsigned prev = atomicAdd(a.done, 1u);
    if (prev == gridDim.x - 1) {  // last CTA of this launch: every store of this rank has been issued and fenced
      *reinterpret_cast<volatile uint32_t*>(a.done) = 0u;
      const uint32_t e = s_epoch;
      __threadfence_system();
      for (int k = 0; k < a.world; ++k) st_release_sys(a.flags_of[k] + 1 * kMaxRanks + a.rank, e);
      const bool ok = wait_all_ranks(a.flags_of[a.rank] + 1 * kMaxRanks, a.world, e);
      if (!ok) atomicCAS(&g_dp_status, 0, 2);
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = e;
      __threadfence();
    }
  }
}

// 'DPAD' payload: the Adam payload <ffff fI> followed by <i> slot (index of this op's flag block).
constexpr uint32_t kSchemaDpAdam = 0x44415044u;  // 'DPAD' little-endian
struct DpAttrs {
  AdamHyper h;
  int32_t slot;
};
bool read_dp_attrs(const void* attr, DpAttrs* out) {
  const AttrBlob& b = blob_of(attr);
  if (b.schema_id != kSchemaDpAdam || !b.data || b.bytes < 28) return false;
  std::memcpy(&out->h, b.data, 24);
  std::memcpy(&out->slot, static_cast<const uint8_t*>(b.data) + 24, 4);
  return out->slot >= 0 && out->slot < kMaxSlots;
}

bool f32_contig(const TensorDesc& d) { return d.dtype == DType::kF32 && d.contiguous && d.rank() >= 1; }

// inputs [P, G, M, V, step(i32)] -> outputs [P, M, V] (biases: P itself is replicated) or [P, M, V, P_lp]
bool dp_adam_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  if (!in || !out || ni != 5 || (no != 3 && no != 4)) return false;
  for (int i = 0; i < 4; ++i)
    if (!f32_contig(in[i]) || !same_shape(in[0], in[i])) return false;
  if (in[4].dtype != DType::kI32 || in[4].numel() != 1) return false;
  // in place only: the op owns a shard, an out-of-place form would leave the other shards undefined
  if (out[0].data != in[0].data || out[1].data != in[2].data || out[2].data != in[3].data) return false;
  for (int i = 0; i < 3; ++i)
    if (!f32_contig(out[i]) || !same_shape(in[0], out[i])) return false;
  if (no == 4) {
    if ((out[3].dtype != DType::kBF16 && out[3].dtype != DType::kF16) || !out[3].contiguous || !same_shape(in[0], out[3]))
      return false;
  }
  if (in[1].data == in[0].data || in[1].data == in[2].data || in[1].data == in[3].data) return false;
  DpAttrs a;
  return read_dp_attrs(attr, &a);
}
bool dp_adam_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  return dp_adam_check(in, ni, out, no, attr);
}

Status dp_adam_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                      cudaStream_t stream) {
  if (!dp_adam_check(in, ni, out, no, attr)) return Status::InvalidArgument;
  DpAttrs at;
  read_dp_attrs(attr, &at);
  const int64_t n = in[0].numel();
  const size_t gbytes = static_cast<size_t>(n) * 4;
  const int bcast_kind = no == 4 ? (out[3].dtype == DType::kBF16 ? 1 : 2) : 3;
  void* bcast_mine = no == 4 ? out[3].data : in[0].data;
  const size_t bbytes = static_cast<size_t>(n) * (bcast_kind == 3 ? 4 : 2);

  DpAdamArgs a{};
  {
    std::lock_guard<std::mutex> lock(g_pools_mu);
    const PeerPool* gp = pool_of(in[1].data, gbytes);
    const PeerPool* bp = pool_of(bcast_mine, bbytes);
    if (!gp || !bp || gp->world != bp->world || gp->rank != bp->rank) return Status::InvalidArgument;  // not peer-visible
    a.rank = gp->rank;
    a.world = gp->world;
    const size_t goff = static_cast<const uint8_t*>(in[1].data) - gp->mine;
    const size_t boff = static_cast<uint8_t*>(bcast_mine) - bp->mine;
    for (int k = 0; k < a.world; ++k) {
      uint8_t* gbase = k == a.rank ? gp->mine : gp->peer[k];
      uint8_t* bbase = k == a.rank ? bp->mine : bp->peer[k];
      if (!gbase || !bbase) return Status::InvalidArgument;
      a.g_of[k] = reinterpret_cast<const float*>(gbase + goff);
      a.bcast_to[k] = bbase + boff;
      a.flags_of[k] = reinterpret_cast<uint32_t*>(gbase) + static_cast<size_t>(at.slot) * 2 * kMaxRanks;
    }
    a.epoch = reinterpret_cast<uint32_t*>(gp->mine + kFlagsBytes) + at.slot;
    a.done = reinterpret_cast<uint32_t*>(gp->mine + kFlagsBytes) + kMaxSlots + at.slot;
  }
  const void* must_align[] = {in[0].data, in[1].data, in[2].data, in[3].data, bcast_mine};
  for (const void* q : must_align)
    if (!aligned_to(q, 16)) return Status::InvalidArgument;
  a.p = static_cast<float*>(in[0].data);
  a.m = static_cast<float*>(in[2].data);
  a.v = static_cast<float*>(in[3].data);
  a.step = static_cast<const int32_t*>(in[4].data);
  a.h = at.h;
  a.bcast_kind = bcast_kind;
  // shard [begin, end): multiples of 4 elements so that packets never straddle two owners
  const int64_t packets = (n + 3) / 4;
  a.begin = std::min<int64_t>(n, (packets * a.rank / a.world) * 4);
  a.end = std::min<int64_t>(n, (packets * (a.rank + 1) / a.world) * 4);
  // One CTA per SM at most: 256 threads x 80 registers fit beside a persistent GEMM CTA (192 x 136), two would not,
  // and a GEMM launched while this kernel is resident must still find room on every SM.
  const int grid = streaming_grid((a.end - a.begin) / 4 + 1, 256, 1);
  // The SM's L1/shared split is one setting for all resident CTAs. The GEMMs run with the largest shared-memory
  // split; asking for the same split here lets these CTAs and GEMM CTAs join each other's SMs in either order
  // (with the default split, a GEMM CTA would have to wait for the SM to drain first).
  static bool carveout_set = false;
  if (!carveout_set) {
    cudaFuncSetAttribute(dp_adam_kernel<1>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(dp_adam_kernel<2>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(dp_adam_kernel<3>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    carveout_set = true;
  }
  cudaGetLastError();
  switch (bcast_kind) {
    case 1: dp_adam_kernel<1><<<grid, 256, 0, stream>>>(a); break;
    case 2: dp_adam_kernel<2><<<grid, 256, 0, stream>>>(a); break;
    default: dp_adam_kernel<3><<<grid, 256, 0, stream>>>(a); break;
  }
  return launch_status();
}

size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }

}  // namespace

KernelVariant make_dp_adam_step_variant() {
  KernelVariant v{};
  v.name = "dp_adam_step_p2p_sm100";
  v.flags = kKV_CaptureSafe;
  v.expected_attr_schema_id = kSchemaDpAdam;
  v.launch = dp_adam_launch;
  v.supported = dp_adam_supported;
  v.query_workspace = no_workspace;
  return v;
}

// ---- peer pool registry (used by the plan) --------------------------------------------------------------
size_t dp_control_bytes() { return kControlBytes; }

bool dp_register_pool(void* mine, size_t bytes, void* const* peers, int rank, int world) {
  if (!mine || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || bytes < kControlBytes) return false;
  PeerPool pp;
  pp.mine = static_cast<uint8_t*>(mine);
  pp.bytes = bytes;
  pp.rank = rank;
  pp.world = world;
  for (int k = 0; k < world; ++k) pp.peer[k] = k == rank ? pp.mine : static_cast<uint8_t*>(peers[k]);
  std::lock_guard<std::mutex> lock(g_pools_mu);
  g_pools.push_back(pp);
  return true;
}

void dp_unregister_pool(void* mine) {
  std::lock_guard<std::mutex> lock(g_pools_mu);
  for (size_t i = 0; i < g_pools.size(); ++i)
    if (g_pools[i].mine == mine) {
      g_pools.erase(g_pools.begin() + static_cast<std::ptrdiff_t>(i));
      return;
    }
}

int dp_wait_status(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_dp_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (clear && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_dp_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace aicf::cuda
