#pragma once
// Shared host/device helpers for the sm_100a kernels of this backend.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <type_traits>

#include "aicf/backends/cuda/registry/attr_blob.hpp"
#include "aicf/backends/cuda/registry/kernel_variant.hpp"
#include "aicf/backends/cuda/registry/status.hpp"
#include "aicf/backends/cuda/registry/tensor_desc.hpp"

namespace aicf::cuda {

// ------------------------------------------------------------------ host helpers
inline Status status_of(cudaError_t e) { return e == cudaSuccess ? Status::Ok : Status::Internal; }
inline Status launch_status() { return status_of(cudaGetLastError()); }

inline const AttrBlob& blob_of(const void* attr) {
  static const AttrBlob kEmpty{};
  return attr ? *static_cast<const AttrBlob*>(attr) : kEmpty;
}

// Copies `n` payload bytes into `dst` when the blob carries schema `want` (or schema 0 when
// `allow_zero_schema`) and at least `n` bytes. Returns false otherwise and leaves dst untouched.
inline bool read_attr_payload(const void* attr, uint32_t want, bool allow_zero_schema, void* dst, size_t n) {
  const AttrBlob& b = blob_of(attr);
  const bool schema_ok = (b.schema_id == want) || (allow_zero_schema && b.schema_id == 0);
  if (!schema_ok || !b.data || b.bytes < n) return false;
  std::memcpy(dst, b.data, n);
  return true;
}

inline bool same_shape(const TensorDesc& a, const TensorDesc& b) {
  if (a.rank() != b.rank()) return false;
  for (int i = 0; i < a.rank(); ++i)
    if (a.shape[i] != b.shape[i]) return false;
  return true;
}

// Product of the extents; false when a dimension is non-positive or rank < min_rank.
inline bool positive_numel(const TensorDesc& t, int min_rank, int64_t* out) {
  if (t.rank() < min_rank || t.rank() > kMaxRank) return false;
  int64_t n = 1;
  for (int i = 0; i < t.rank(); ++i) {
    if (t.shape[i] <= 0) return false;
    n *= t.shape[i];
  }
  *out = n;
  return true;
}

// [..., N] viewed as [M, N]; needs rank >= 2 and positive extents.
inline bool rows_cols_lastdim(const TensorDesc& t, int64_t* M, int64_t* N) {
  const int r = t.rank();
  if (r < 2 || r > kMaxRank) return false;
  int64_t m = 1;
  for (int i = 0; i < r - 1; ++i) {
    if (t.shape[i] <= 0) return false;
    m *= t.shape[i];
  }
  if (t.shape[r - 1] <= 0) return false;
  *M = m;
  *N = t.shape[r - 1];
  return true;
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Per-device state (SM counts, function attributes, shared-memory carveouts and symbol addresses are properties of
// one device, not of the process) lives in tables of kMaxDevices slots indexed by the CUDA device ordinal.
constexpr int kMaxDevices = 64;

// Ordinal of the current device, or -1 when it does not fit the per-device tables (such a device still works: the
// callers then redo their one-time set-up on every call instead of caching it).
inline int device_slot() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return dev >= 0 && dev < kMaxDevices ? dev : -1;
}

// One "set-up done" flag per device. Set-up bodies are idempotent (cudaFuncSetAttribute and the like), so two threads
// that both find the flag clear may both run them; the flags are atomics so that this is not a data race.
struct PerDeviceOnce {
  std::atomic<int> done[kMaxDevices] = {};
  // Runs fn() (returning true on success) unless it already succeeded on the current device.
  template <typename Fn> bool run(Fn&& fn) {
    const int dev = device_slot();
    if (dev >= 0 && done[dev].load(std::memory_order_acquire)) return true;
    if (!fn()) return false;
    if (dev >= 0) done[dev].store(1, std::memory_order_release);
    return true;
  }
};

// Number of SMs of the current device (148 on B200); cached per device.
inline int sm_count() {
  static std::atomic<int> cached[kMaxDevices] = {};
  const int dev = device_slot();
  if (dev >= 0) {
    const int c = cached[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int cur = 0, n = 0;
  cudaGetDevice(&cur);
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, cur) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 148;
  }
  if (dev >= 0) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// Blocks per SM for kernels that only stream through arrays (element-wise ops, casts, optimizers, last-axis
// reductions): as many blocks as the array needs at a few packets per thread, far more than an SM holds at once,
// rather than a resident grid with a long grid-stride loop. Measured with fused Adam on 2^28 elements, 256-thread
// blocks per SM -> GB/s: 4 (all resident) 5983, 32 6421, 128 6615, 512 6857, 768 6919, 1024 6911; a copy-like probe
// kernel follows the same curve for four reads + three writes and for one read + one write (6351-6458 at 32, 6900 at
// 512-1024).
constexpr int kStreamBlocksPerSm = 768;

// Grid for a grid-stride streaming kernel: whole multiples of the SM count, no more blocks than
// there is work, at least one.
inline int streaming_grid(int64_t work_items, int items_per_block, int blocks_per_sm) {
  int64_t need = (work_items + items_per_block - 1) / items_per_block;
  if (need < 1) need = 1;
  const int64_t cap = static_cast<int64_t>(sm_count()) * blocks_per_sm;
  return static_cast<int>(need < cap ? need : cap);
}

// ------------------------------------------------------------------ device helpers
#ifdef __CUDACC__

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  __device__ __forceinline__ static float to_f(float v) { return v; }
  __device__ __forceinline__ static float from_f(float v) { return v; }
};
template <> struct Cvt<__half> {
  __device__ __forceinline__ static float to_f(__half v) { return __half2float(v); }
  __device__ __forceinline__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
  __device__ __forceinline__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte packet of T with float unpack/pack.
template <typename T> struct alignas(16) Pack16 {
  static constexpr int kN = 16 / sizeof(T);
  T v[kN];
};

// A packet to / from its kN floats. Same values as converting element by element (round to nearest even), but the
// 16-bit types convert two elements per instruction: bf16 -> f32 is a shift or a mask of the 32-bit word,
// f32 -> bf16 / f16 one cvt.rn.{bf16x2,f16x2}.f32 per pair. The 16-bit row kernels are bound by instruction issue,
// not by HBM, so the conversions are where their time goes.
template <typename T>
__device__ __forceinline__ void unpack16(const Pack16<T>& p, float (&f)[Pack16<T>::kN]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < Pack16<T>::kN; ++e) f[e] = Cvt<T>::to_f(p.v[e]);
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  } else {
    const __half2* h = reinterpret_cast<const __half2*>(&p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}
template <typename T>
__device__ __forceinline__ void pack16(Pack16<T>& o, const float (&f)[Pack16<T>::kN]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < Pack16<T>::kN; ++e) o.v[e] = Cvt<T>::from_f(f[e]);
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    __nv_bfloat162* w = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  } else {
    __half2* w = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
}

// Streaming (evict-first) 16-byte global accesses: data touched once should not displace L2 lines.
template <typename T>
__device__ __forceinline__ Pack16<T> ld_stream(const Pack16<T>* p) {
  const int4 raw = __ldcs(reinterpret_cast<const int4*>(p));
  Pack16<T> out;
  *reinterpret_cast<int4*>(&out) = raw;
  return out;
}
template <typename T>
__device__ __forceinline__ void st_stream(Pack16<T>* p, const Pack16<T>& v) {
  __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

#endif  // __CUDACC__

}  // namespace aicf::cuda
