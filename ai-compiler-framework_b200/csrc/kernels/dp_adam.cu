// Data-parallel optimizer step fused with its gradient exchange, over NVLink peer memory.
//
// One launch per parameter tensor and rank does what all_reduce + adam_step + weight broadcast would do:
//   1. tells every peer "my gradient of this tensor is final and nobody here reads the old weights any more"
//      and waits for the same word from all of them (flags in peer-visible memory, sequence numbers, no reset);
//   2. for ITS shard of the tensor (elements [n*r/N, n*(r+1)/N), 4-aligned): sums the N shard gradients straight
//      out of the peers' gradient buffers (P2P loads, always in rank order 0..N-1, so the sum is bit-reproducible),
//      applies Adam to its shard of the fp32 master weights and moments, and stores the new weights into every
//      rank's working copy (bf16 / f16 copy for matrices, the fp32 parameter itself for biases) with P2P stores;
//   3. tells every peer "my stores into your memory are done". The last CTA then waits for the same word from all
//      peers, so kernel completion means this rank's working copies are complete and its gradient buffer may be
//      overwritten - or, when the op carries `defer_done`, leaves that wait to the op of the step that carries
//      `fence_slots` (the last exchange of the step waits for the done words of every slot): nothing inside a step
//      reads a working copy or rewrites a gradient after its exchange, so one rendezvous at the end of the step
//      replaces one per tensor and the exchanges of a step run back to back.
// Reduce-scatter, update and all-gather travel over NVLink once each (4 B/param in, 2 B/param out per rank for
// matrices) and Adam's 28 B/param of HBM traffic shrinks to 1/N per rank. Peer loads are latency-bound, so every
// thread keeps the gradient packets of several iterations in flight (at least eight remote 16-byte loads per thread
// whatever the number of ranks). The kernel uses a few bytes of shared memory and at most 144 registers x 256
// threads, so its CTAs co-reside with the persistent GEMM CTAs of the backward pass (192 threads x 136 registers)
// instead of waiting for SMs.
//
// fp32 master weights and moments of matrices are therefore sharded: rank r's copy is current only inside its
// shard (gather the shards to read a whole master tensor). Working copies and biases are complete on every rank.
//
// Waits are bounded (~2 s). The ready-phase wait is made by ONE thread of the launch (CTA 0), which publishes go or
// no-go for all CTAs: either every CTA updates and broadcasts its part of the shard or none does, so a peer that
// arrives around the limit cannot leave a tensor half updated. A wait that expires sets a status word
// (aicf_b200_wait_status bits 17-18), skips the work that depended on it and lets the kernel finish; after a
// non-zero status the replicas are no longer known to agree and training has to resume from a checkpoint.
// No TMA multicast, no multimem: plain peer loads and stores.
#include <algorithm>
#include <mutex>
#include <string>
#include <type_traits>
#include <vector>

#include "../capi/capi_internal.hpp"
#include "adam_math.cuh"

namespace aicf::cuda {

constexpr int kMaxRanks = 8;
constexpr int kMaxSlots = 60;  // dp_adam_step ops per plan
// Layout of the control block at the start of every peer pool (8 KiB):
//   uint32 flags[kMaxSlots][2][kMaxRanks]   written by peers (phase 0 = ready, phase 1 = done)
//   uint32 epoch[kMaxSlots]; uint32 done[kMaxSlots]; uint32 go[kMaxSlots]   local
constexpr size_t kFlagsBytes = size_t(kMaxSlots) * 2 * kMaxRanks * 4;
constexpr size_t kControlBytes = 8192;
static_assert(kFlagsBytes + size_t(kMaxSlots) * 12 <= kControlBytes, "control block layout");

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
  uint32_t *epoch, *done, *go;  // this op's words in the local control block
  int64_t begin, end;  // this rank's shard
  int rank, world;
  int bcast_kind;  // 1 bf16, 2 f16, 3 fp32 (the parameter itself)
  int defer_done;  // 1: do not wait for the peers' done words here
  int fence_slots;  // > 0: before finishing, wait for the done words of slots [0, fence_slots) of this pool
  const uint32_t* flags_base;  // flag blocks of all slots in the local pool (fence)
  const uint32_t* epoch_base;  // epoch words of all slots in the local pool (fence)
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

__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// kUnroll packets per thread at a time, kW gradient sources each: every load (kUnroll x kW gradient packets, most of
// them over NVLink, and the local p, m, v packets) is issued before the first one is used.
template <int kBcast, int kW, int kUnroll>
__device__ __forceinline__ void update_packets(const DpAdamArgs& a, int world, int64_t i, int64_t stride, float d1, float d2) {
  using V4 = Pack16<float>;
  float4 gk[kUnroll][kW];
  V4 p[kUnroll], m[kUnroll], v[kUnroll];
#pragma unroll
  for (int u = 0; u < kUnroll; ++u)
#pragma unroll
    for (int k = 0; k < kW; ++k)
      if (k < world) gk[u][k] = __ldcg(reinterpret_cast<const float4*>(a.g_of[k]) + (i + u * stride));
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    p[u] = ld_stream(reinterpret_cast<const V4*>(a.p) + (i + u * stride));
    m[u] = ld_stream(reinterpret_cast<const V4*>(a.m) + (i + u * stride));
    v[u] = ld_stream(reinterpret_cast<const V4*>(a.v) + (i + u * stride));
  }
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    float4 acc = gk[u][0];
#pragma unroll
    for (int k = 1; k < kW; ++k)  // fixed rank order: the same bits whoever owns the shard
      if (k < world) {
        acc.x += gk[u][k].x;
        acc.y += gk[u][k].y;
        acc.z += gk[u][k].z;
        acc.w += gk[u][k].w;
      }
    const float g[4] = {acc.x, acc.y, acc.z, acc.w};
    V4 po, mo, vo;
#pragma unroll
    for (int e = 0; e < 4; ++e) adam_one<false>(p[u].v[e], g[e], m[u].v[e], v[u].v[e], a.h, d1, d2, po.v[e], mo.v[e], vo.v[e]);
    const int64_t at = i + u * stride;
    st_stream(reinterpret_cast<V4*>(a.m) + at, mo);
    st_stream(reinterpret_cast<V4*>(a.v) + at, vo);
    if (kBcast != 3) st_stream(reinterpret_cast<V4*>(a.p) + at, po);
    bcast_x4<kBcast>(a, at, po);
  }
}

// kWorld: 2, 4 or 8 ranks with the loops over ranks unrolled to exactly that count, or 0 = any count up to
// kMaxRanks (predicated). kUnroll: packets per thread per iteration.
template <int kBcast, int kWorld, int kUnroll>
__global__ void __launch_bounds__(256) dp_adam_kernel(const DpAdamArgs a) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_go;
  if (threadIdx.x == 0) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.epoch) + 1u;
    s_epoch = e;
    // go word of this launch: low 31 bits = the epoch it answers for, top bit = no-go
    const uint32_t tag = e & 0x7FFFFFFFu;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int k = 0; k < a.world; ++k) st_release_sys(a.flags_of[k] + 0 * kMaxRanks + a.rank, e);
      const bool ok = wait_all_ranks(a.flags_of[a.rank] + 0 * kMaxRanks, a.world, e);
      if (!ok) atomicCAS(&g_dp_status, 0, 1);
      st_release_gpu(a.go, ok ? tag : (tag | 0x80000000u));
      s_go = ok ? 1 : 0;
    } else {
      // CTA 0 is dispatched before any other CTA of the grid, so it is resident whenever this one is
      const unsigned long long t0 = now_ns();
      uint32_t spin = 0, w;
      bool answered = true;
      while (((w = ld_acquire_gpu(a.go)) & 0x7FFFFFFFu) != tag) {
        if ((++spin & 63u) == 0u && now_ns() - t0 > kPeerWaitBudgetNs + kPeerWaitBudgetNs / 2) {
          answered = false;
          break;
        }
      }
      if (!answered) atomicCAS(&g_dp_status, 0, 1);
      s_go = (answered && (w >> 31) == 0u) ? 1 : 0;
    }
  }
  __syncthreads();

  if (s_go) {
    float d1, d2;
    adam_inverse_corrections(a.h, a.step[0], d1, d2);
    constexpr int kW = kWorld ? kWorld : kMaxRanks;
    const int world = kWorld ? kWorld : a.world;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // shard bounds are multiples of 4 except possibly the very end of the tensor
    const int64_t p_begin = a.begin >> 2, p_end = a.end >> 2;
    int64_t i = p_begin + tid;
    for (; i + (kUnroll - 1) * stride < p_end; i += kUnroll * stride) update_packets<kBcast, kW, kUnroll>(a, world, i, stride, d1, d2);
    for (; i < p_end; i += stride) update_packets<kBcast, kW, 1>(a, world, i, stride, d1, d2);
    for (int64_t j = (p_end << 2) + tid; j < a.end; j += stride) {  // ragged end of the last shard
      float g = __ldcg(a.g_of[0] + j);
      for (int k = 1; k < a.world; ++k) g += __ldcg(a.g_of[k] + j);
      float po, mo, vo;
      adam_one<false>(a.p[j], g, a.m[j], a.v[j], a.h, d1, d2, po, mo, vo);
      a.m[j] = mo;
      a.v[j] = vo;
      if (kBcast != 3) a.p[j] = po;
      bcast_x1<kBcast>(a, j, po);
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
      *reinterpret_cast<volatile uint32_t*>(a.epoch) = e;
      __threadfence();
      bool ok = true;
      if (!a.defer_done) ok = wait_all_ranks(a.flags_of[a.rank] + 1 * kMaxRanks, a.world, e);
      // step-end fence: the done words of every slot of this pool, each against that slot's own epoch (slots
      // that were launched earlier on this stream have published theirs; unused slots read 0 >= 0)
      for (int sl = 0; ok && sl < a.fence_slots; ++sl) {
        const uint32_t es = *reinterpret_cast<const volatile uint32_t*>(a.epoch_base + sl);
        ok = wait_all_ranks(a.flags_base + (static_cast<size_t>(sl) * 2 + 1) * kMaxRanks, a.world, es);
      }
      if (!ok) atomicCAS(&g_dp_status, 0, 2);
    }
  }
}

// 'DPAD' payload: the Adam payload <ffff fI> followed by <i> slot (index of this op's flag block) and, optionally,
// <ii> flags (bit 0 defer_done: leave the done-phase wait to the step's fence; bit 1 solo: no other kernel runs beside
// this op, take two CTAs per SM), fence_slots (> 0: this op is the fence).
constexpr uint32_t kSchemaDpAdam = 0x44415044u;  // 'DPAD' little-endian
struct DpAttrs {
  AdamHyper h;
  int32_t slot;
  int32_t defer_done = 0;
  int32_t fence_slots = 0;
};
bool read_dp_attrs(const void* attr, DpAttrs* out) {
  const AttrBlob& b = blob_of(attr);
  if (b.schema_id != kSchemaDpAdam || !b.data || b.bytes < 28) return false;
  std::memcpy(&out->h, b.data, 24);
  std::memcpy(&out->slot, static_cast<const uint8_t*>(b.data) + 24, 4);
  out->defer_done = out->fence_slots = 0;
  if (b.bytes >= 36) {
    std::memcpy(&out->defer_done, static_cast<const uint8_t*>(b.data) + 28, 4);
    std::memcpy(&out->fence_slots, static_cast<const uint8_t*>(b.data) + 32, 4);
  }
  if (out->fence_slots < 0 || out->fence_slots > kMaxSlots) return false;
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
    a.go = reinterpret_cast<uint32_t*>(gp->mine + kFlagsBytes) + 2 * kMaxSlots + at.slot;
    a.flags_base = reinterpret_cast<const uint32_t*>(gp->mine);
    a.epoch_base = reinterpret_cast<const uint32_t*>(gp->mine + kFlagsBytes);
  }
  a.defer_done = (at.defer_done & 1) ? 1 : 0;
  a.fence_slots = at.fence_slots;
  const bool solo = (at.defer_done & 2) != 0;  // nothing runs beside this op: no need to leave room for GEMM CTAs
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
  // One CTA per SM at most: 256 threads x (at most) 144 registers fit beside a persistent GEMM CTA (192 x 136), two
  // would not, and a GEMM launched while this kernel is resident must still find room on every SM.
  // An op marked `solo` (the step's last exchange, which has no GEMM left to overlap with) takes two CTAs per SM, all
  // the register file allows: twice the peer loads in flight, which is what bounds a kernel that waits on NVLink.
  const int grid = streaming_grid((a.end - a.begin) / 4 + 1, 256, solo ? 2 : 1);
  // The SM's L1/shared split is one setting for all resident CTAs. The GEMMs run with the largest shared-memory
  // split; asking for the same split here lets these CTAs and GEMM CTAs join each other's SMs in either order
  // (with the default split, a GEMM CTA would have to wait for the SM to drain first).
  // Ranks unrolled for 2, 4 and 8 (predicated loop otherwise); packets per thread chosen so that at least eight
  // remote loads are in flight per thread.
  auto launch = [&](auto bc, auto wd, auto un) {
    constexpr int kB = decltype(bc)::value, kWd = decltype(wd)::value, kUn = decltype(un)::value;
    static PerDeviceOnce carveout;  // a per-device function attribute
    carveout.run([] {
      cudaFuncSetAttribute(dp_adam_kernel<kB, kWd, kUn>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      return true;
    });
    cudaGetLastError();
    dp_adam_kernel<kB, kWd, kUn><<<grid, 256, 0, stream>>>(a);
  };
  auto by_world = [&](auto bc) {
    using I = std::integral_constant<int, 0>;
    switch (a.world) {
      case 2: launch(bc, std::integral_constant<int, 2>{}, std::integral_constant<int, 4>{}); break;
      case 4: launch(bc, std::integral_constant<int, 4>{}, std::integral_constant<int, 3>{}); break;
      case 8: launch(bc, std::integral_constant<int, 8>{}, std::integral_constant<int, 2>{}); break;
      default: launch(bc, I{}, std::integral_constant<int, 1>{}); break;
    }
  };
  switch (bcast_kind) {
    case 1: by_world(std::integral_constant<int, 1>{}); break;
    case 2: by_world(std::integral_constant<int, 2>{}); break;
    default: by_world(std::integral_constant<int, 3>{}); break;
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
