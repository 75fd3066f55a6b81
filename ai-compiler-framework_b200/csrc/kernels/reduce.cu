// Reductions, all in a fixed summation order (no atomics) so results are bit-reproducible:
//   * column sum  [M,N] -> [N]   ("keep last dim": the bias gradient; reference ops/reduce_sum)
//   * last-axis sum / max / mean  [M,N] -> [M]
//
// Column sum layout: a block is 32 column-lanes x 8 row-lanes. A column-lane owns one 16-byte packet
// of adjacent columns, so every warp load is a fully coalesced 512-byte row segment (the reference
// gives a column to a whole block and reads it with stride N). Rows are split over gridDim.y so the
// grid fills the SMs; with more than one split the per-split partial sums go to a scratch buffer
// [splits, N] (fp32) and a second kernel adds them in split order.
#include <cstdlib>
#include <mutex>
#include <string>

#include "../capi/capi_internal.hpp"
#include "common.cuh"

namespace aicf::cuda {

namespace {

constexpr int kColLanes = 32;
constexpr int kRowLanes = 8;

struct ColPlan {
  int64_t M = 0, N = 0;
  int vec = 1;         // elements per column-lane
  int64_t col_blocks = 0;
  int splits = 1;
  int64_t rows_per_split = 0;
};

template <typename T>
ColPlan plan_columns(int64_t M, int64_t N, bool aligned) {
  ColPlan p;
  p.M = M;
  p.N = N;
  constexpr int kN = Pack16<T>::kN;
  p.vec = (aligned && N % kN == 0) ? kN : 1;
  const int64_t cols_per_block = static_cast<int64_t>(kColLanes) * p.vec;
  p.col_blocks = (N + cols_per_block - 1) / cols_per_block;
  const int64_t want_blocks = static_cast<int64_t>(sm_count()) * 4;
  int64_t s = (want_blocks + p.col_blocks - 1) / p.col_blocks;
  const int64_t max_s = (M + 63) / 64;  // at least 64 rows per split
  if (s > max_s) s = max_s;
  if (s < 1) s = 1;
  if (s > 65535) s = 65535;
  p.rows_per_split = (M + s - 1) / s;
  p.splits = static_cast<int>((M + p.rows_per_split - 1) / p.rows_per_split);
  return p;
}

template <typename T, int kVec, typename OutT>
__global__ void __launch_bounds__(kColLanes* kRowLanes)
    colsum_kernel(const T* __restrict__ x, OutT* __restrict__ out, float* __restrict__ partial, int64_t M, int64_t N,
                  int64_t rows_per_split, int splits) {
  __shared__ float red[kRowLanes][kColLanes * kVec + 1];
  const int cx = threadIdx.x % kColLanes;
  const int ry = threadIdx.x / kColLanes;
  const int64_t col0 = (static_cast<int64_t>(blockIdx.x) * kColLanes + cx) * kVec;
  const int64_t r_begin = static_cast<int64_t>(blockIdx.y) * rows_per_split;
  int64_t r_end = r_begin + rows_per_split;
  if (r_end > M) r_end = M;

  float acc[kVec];
#pragma unroll
  for (int e = 0; e < kVec; ++e) acc[e] = 0.0f;

  if (col0 < N) {
    int64_t r = r_begin + ry;
    if (kVec > 1) {
      using PK = Pack16<T>;
      // 4 rows in flight per thread
      for (; r + 3 * kRowLanes < r_end; r += 4 * kRowLanes) {
        PK p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) p[u] = ld_stream(reinterpret_cast<const PK*>(x + (r + u * kRowLanes) * N + col0));
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < kVec; ++e) acc[e] += Cvt<T>::to_f(p[u].v[e]);
      }
      for (; r < r_end; r += kRowLanes) {
        const PK p = ld_stream(reinterpret_cast<const PK*>(x + r * N + col0));
#pragma unroll
        for (int e = 0; e < kVec; ++e) acc[e] += Cvt<T>::to_f(p.v[e]);
      }
    } else {
      for (; r < r_end; r += kRowLanes) acc[0] += Cvt<T>::to_f(x[r * N + col0]);
    }
  }
#pragma unroll
  for (int e = 0; e < kVec; ++e) red[ry][cx * kVec + e] = acc[e];
  __syncthreads();
  // row-lane 0 folds the 8 row-lane partials in order
  if (ry == 0 && col0 < N) {
#pragma unroll
    for (int e = 0; e < kVec; ++e) {
      float s = red[0][cx * kVec + e];
#pragma unroll
      for (int y = 1; y < kRowLanes; ++y) s += red[y][cx * kVec + e];
      if (splits == 1) {
        out[col0 + e] = Cvt<OutT>::from_f(s);
      } else {
        partial[static_cast<int64_t>(blockIdx.y) * N + col0 + e] = s;
      }
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256) colsum_finish_kernel(const float* __restrict__ partial, OutT* __restrict__ out,
                                                           int64_t N, int splits) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = partial[c];
  for (int k = 1; k < splits; ++k) s += partial[static_cast<int64_t>(k) * N + c];
  out[c] = Cvt<OutT>::from_f(s);
}

int64_t read_axis(const void* attr) {
  int64_t axis = 0;
  read_attr_payload(attr, schema::kReduceSum, true, &axis, 8);
  return axis;
}

// Contract of the reference ids (ops/reduce_sum/launcher.cu:240-312): one contiguous input of rank
// >= 2, axis attr 0 (or absent), output a contiguous vector of length N = last extent.
template <DType kIn, DType kOut>
bool colsum_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != kIn || !in[0].contiguous || in[0].rank() < 2) return false;
  if (read_axis(attr) != 0) return false;
  int64_t M = 0, N = 0;
  if (!rows_cols_lastdim(in[0], &M, &N)) return false;
  return out[0].dtype == kOut && out[0].contiguous && out[0].rank() == 1 && out[0].shape[0] == N;
}
template <DType kIn, DType kOut>
bool colsum_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  return colsum_check<kIn, kOut>(in, ni, out, no, attr);
}
template <typename T>
size_t colsum_workspace(const TensorDesc* in, int ni, const void*) {
  if (!in || ni != 1) return 0;
  int64_t M = 0, N = 0;
  if (!rows_cols_lastdim(in[0], &M, &N)) return 0;
  const ColPlan p = plan_columns<T>(M, N, aligned_to(in[0].data, 16));
  return p.splits > 1 ? static_cast<size_t>(p.splits) * static_cast<size_t>(N) * sizeof(float) : 0;
}

template <typename T, typename OutT>
Status colsum_run(const T* x, OutT* out, int64_t M, int64_t N, void* ws, size_t ws_bytes, cudaStream_t stream) {
  const ColPlan p = plan_columns<T>(M, N, aligned_to(x, 16));
  float* partial = nullptr;
  if (p.splits > 1) {
    const size_t need = static_cast<size_t>(p.splits) * static_cast<size_t>(N) * sizeof(float);
    if (!ws || ws_bytes < need) return Status::InvalidArgument;
    partial = static_cast<float*>(ws);
  }
  const dim3 grid(static_cast<unsigned>(p.col_blocks), static_cast<unsigned>(p.splits));
  cudaGetLastError();
  if (p.vec > 1) {
    colsum_kernel<T, Pack16<T>::kN, OutT><<<grid, kColLanes * kRowLanes, 0, stream>>>(x, out, partial, M, N,
                                                                                   p.rows_per_split, p.splits);
  } else {
    colsum_kernel<T, 1, OutT><<<grid, kColLanes * kRowLanes, 0, stream>>>(x, out, partial, M, N, p.rows_per_split,
                                                                         p.splits);
  }
  if (p.splits > 1) {
    colsum_finish_kernel<OutT><<<static_cast<unsigned>((N + 255) / 256), 256, 0, stream>>>(partial, out, N, p.splits);
  }
  return launch_status();
}

template <DType kIn, DType kOut, typename T, typename OutT>
Status colsum_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void* ws, size_t ws_bytes,
                     cudaStream_t stream) {
  if (!colsum_check<kIn, kOut>(in, ni, out, no, attr)) return Status::InvalidArgument;
  int64_t M = 0, N = 0;
  rows_cols_lastdim(in[0], &M, &N);
  return colsum_run<T, OutT>(static_cast<const T*>(in[0].data), static_cast<OutT*>(out[0].data), M, N, ws, ws_bytes,
                             stream);
}

// ------------------------------------------------------------------------------------------------
// Last-axis reductions: one warp per row; a lane walks packets lane, lane+32, ... with four packets
// in flight, keeps one accumulator per packet element, folds them in element order, then a butterfly
// shuffle finishes the row. Rows that are not 16-byte aligned take the scalar walk.
// ------------------------------------------------------------------------------------------------
enum class RowOp { Sum, Max, Mean };

template <RowOp kOp> __device__ __forceinline__ float row_identity() { return kOp == RowOp::Max ? -INFINITY : 0.0f; }
template <RowOp kOp> __device__ __forceinline__ float row_combine(float a, float b) {
  return kOp == RowOp::Max ? fmaxf(a, b) : a + b;
}

template <typename T, RowOp kOp>
__global__ void __launch_bounds__(256) rowreduce_kernel(const T* __restrict__ x, float* __restrict__ out, int64_t M,
                                                       int64_t N, int vec_ok) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp; row < M; row += nwarps) {
    const T* xr = x + row * N;
    float acc[kN];
#pragma unroll
    for (int e = 0; e < kN; ++e) acc[e] = row_identity<kOp>();
    if (vec_ok) {
      const int64_t np = N / kN;
      const PK* pr = reinterpret_cast<const PK*>(xr);
      int64_t i = lane;
      for (; i + 96 < np; i += 128) {
        PK p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) p[u] = ld_stream(pr + i + 32 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < kN; ++e) acc[e] = row_combine<kOp>(acc[e], Cvt<T>::to_f(p[u].v[e]));
      }
      for (; i < np; i += 32) {
        const PK p = ld_stream(pr + i);
#pragma unroll
        for (int e = 0; e < kN; ++e) acc[e] = row_combine<kOp>(acc[e], Cvt<T>::to_f(p.v[e]));
      }
    } else {
      for (int64_t i = lane; i < N; i += 32) acc[0] = row_combine<kOp>(acc[0], Cvt<T>::to_f(xr[i]));
    }
    float v = acc[0];
#pragma unroll
    for (int e = 1; e < kN; ++e) v = row_combine<kOp>(v, acc[e]);
    v = kOp == RowOp::Max ? warp_max(v) : warp_sum(v);
    if (lane == 0) out[row] = kOp == RowOp::Mean ? v / static_cast<float>(N) : v;
  }
}

// [..., N] -> [...] f32. Input rank >= 1 (a vector reduces to a scalar-like output of one element).
bool rows_cols_any(const TensorDesc& t, int64_t* M, int64_t* N) {
  const int r = t.rank();
  if (r < 1 || r > kMaxRank) return false;
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
template <DType kIn>
bool rowreduce_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr, bool axis_attr) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != kIn || !in[0].contiguous) return false;
  int64_t M = 0, N = 0;
  if (!rows_cols_any(in[0], &M, &N)) return false;
  if (axis_attr) {  // reduce_sum shares its kind with the column sum: the last-axis form needs axis -1 / rank-1
    const int64_t axis = read_axis(attr);
    if (axis != -1 && axis != in[0].rank() - 1) return false;
    if (in[0].rank() >= 2 && axis == 0) return false;
  }
  if (out[0].dtype != DType::kF32 || !out[0].contiguous) return false;
  int64_t on = 0;
  if (!positive_numel(out[0], 0, &on)) return false;
  return on == M;
}
template <DType kIn, RowOp kOp>
bool rowreduce_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  return rowreduce_check<kIn>(in, ni, out, no, attr, kOp == RowOp::Sum);
}
template <DType kIn, RowOp kOp, typename T>
Status rowreduce_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                        cudaStream_t stream) {
  if (!rowreduce_check<kIn>(in, ni, out, no, attr, kOp == RowOp::Sum)) return Status::InvalidArgument;
  int64_t M = 0, N = 0;
  rows_cols_any(in[0], &M, &N);
  const int vec = aligned_to(in[0].data, 16) && (N % Pack16<T>::kN == 0);
  // AICF_ROWREDUCE_GRID=n (tuning, read once per process): blocks per SM
  static const int per_sm = [] {
    const char* e = std::getenv("AICF_ROWREDUCE_GRID");
    const int v = e ? std::atoi(e) : 0;
    return v >= 1 && v <= 4096 ? v : kStreamBlocksPerSm;
  }();
  const int grid = streaming_grid(M, 8, per_sm);  // 8 warps (rows) per block
  cudaGetLastError();
  rowreduce_kernel<T, kOp><<<grid, 256, 0, stream>>>(static_cast<const T*>(in[0].data),
                                                    static_cast<float*>(out[0].data), M, N, vec);
  return launch_status();
}
size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }

using LaunchFn = Status (*)(const TensorDesc*, int, TensorDesc*, int, const void*, void*, size_t, cudaStream_t);
using SupportedFn = bool (*)(const TensorDesc*, int, const TensorDesc*, int, const void*);
using WorkspaceFn = size_t (*)(const TensorDesc*, int, const void*);
KernelVariant make(const char* name, LaunchFn l, SupportedFn s, WorkspaceFn w) {
  KernelVariant v{};
  v.name = name;
  v.flags = kKV_CaptureSafe;
  v.launch = l;
  v.supported = s;
  v.query_workspace = w;
  return v;
}

}  // namespace

// Column sum entry for callers that bring their own scratch (used by the C ABI's direct entry points).
Status colsum_f32_direct(const float* x, float* out, int64_t M, int64_t N, void* ws, size_t ws_bytes,
                         cudaStream_t stream) {
  return colsum_run<float, float>(x, out, M, N, ws, ws_bytes, stream);
}
size_t colsum_f32_scratch_bytes(const float* x, int64_t M, int64_t N) {
  const ColPlan p = plan_columns<float>(M, N, aligned_to(x, 16));
  return p.splits > 1 ? static_cast<size_t>(p.splits) * static_cast<size_t>(N) * sizeof(float) : 0;
}

KernelVariant make_reduce_sum_lastdim_f32_variant() {
  return make("colsum_f32_sm100", colsum_launch<DType::kF32, DType::kF32, float, float>,
              colsum_supported<DType::kF32, DType::kF32>, colsum_workspace<float>);
}
KernelVariant make_reduce_sum_lastdim_f16_to_f32_variant() {
  return make("colsum_f16_to_f32_sm100", colsum_launch<DType::kF16, DType::kF32, __half, float>,
              colsum_supported<DType::kF16, DType::kF32>, colsum_workspace<__half>);
}
KernelVariant make_reduce_sum_lastdim_f16_variant() {
  return make("colsum_f16_sm100", colsum_launch<DType::kF16, DType::kF16, __half, __half>,
              colsum_supported<DType::kF16, DType::kF16>, colsum_workspace<__half>);
}
KernelVariant make_reduce_sum_lastdim_bf16_to_f32_variant() {
  return make("colsum_bf16_to_f32_sm100", colsum_launch<DType::kBF16, DType::kF32, __nv_bfloat16, float>,
              colsum_supported<DType::kBF16, DType::kF32>, colsum_workspace<__nv_bfloat16>);
}
KernelVariant make_reduce_sum_lastdim_bf16_variant() {
  return make("colsum_bf16_sm100", colsum_launch<DType::kBF16, DType::kBF16, __nv_bfloat16, __nv_bfloat16>,
              colsum_supported<DType::kBF16, DType::kBF16>, colsum_workspace<__nv_bfloat16>);
}

// ------------------------------------------------------------------------------------------------
// Column sum for callers that cannot allocate (aicf_b200_colsum_f32_noalloc).
//
// The per-split partial sums live in a fixed array in device memory that is part of the library
// image: every GPU that loads the library carries these 512 KiB until the process exits, and no
// allocation call is ever made on its behalf. `g_noalloc_scratch` names the array for device code;
// on the host the same name is only a handle for the runtime, so the address kernels receive is
// looked up once per device with cudaGetSymbolAddress while that device is current.
// ------------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = size_t(512) << 10;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchBytes / sizeof(float)];

namespace {
float* g_noalloc_ptr[kMaxDevices] = {nullptr};  // kMaxDevices: the one limit of every per-device table (common.cuh)
std::mutex g_noalloc_mu;

// Device address of the scratch array on the current device (looked up on the first call there).
cudaError_t noalloc_scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return cudaSuccess;
}
}  // namespace

#define AICF_ROWREDUCE(fn, nm, DT, OP, T) \
  KernelVariant fn() { return make(nm, rowreduce_launch<DT, OP, T>, rowreduce_supported<DT, OP>, no_workspace); }
AICF_ROWREDUCE(make_reduce_sum_lastaxis_f32_variant, "rowsum_f32_sm100", DType::kF32, RowOp::Sum, float)
AICF_ROWREDUCE(make_reduce_sum_lastaxis_bf16_variant, "rowsum_bf16_sm100", DType::kBF16, RowOp::Sum, __nv_bfloat16)
AICF_ROWREDUCE(make_reduce_sum_lastaxis_f16_variant, "rowsum_f16_sm100", DType::kF16, RowOp::Sum, __half)
AICF_ROWREDUCE(make_reduce_max_lastaxis_f32_variant, "rowmax_f32_sm100", DType::kF32, RowOp::Max, float)
AICF_ROWREDUCE(make_reduce_max_lastaxis_bf16_variant, "rowmax_bf16_sm100", DType::kBF16, RowOp::Max, __nv_bfloat16)
AICF_ROWREDUCE(make_reduce_max_lastaxis_f16_variant, "rowmax_f16_sm100", DType::kF16, RowOp::Max, __half)
AICF_ROWREDUCE(make_reduce_mean_lastaxis_f32_variant, "rowmean_f32_sm100", DType::kF32, RowOp::Mean, float)
AICF_ROWREDUCE(make_reduce_mean_lastaxis_bf16_variant, "rowmean_bf16_sm100", DType::kBF16, RowOp::Mean, __nv_bfloat16)
AICF_ROWREDUCE(make_reduce_mean_lastaxis_f16_variant, "rowmean_f16_sm100", DType::kF16, RowOp::Mean, __half)

}  // namespace aicf::cuda

extern "C" int aicf_b200_colsum_f32_noalloc(const float* x, float* out, int64_t rows, int64_t cols, aicf_stream stream) {
  using namespace aicf::cuda;
  using aicf::capi::fail;
  if (!x || !out || rows <= 0 || cols <= 0) return fail(Status::InvalidArgument, "colsum_f32_noalloc: null pointer or empty shape");
  const size_t need = colsum_f32_scratch_bytes(x, rows, cols);
  if (need > kNoAllocScratchBytes) {
    return fail(Status::InvalidArgument,
                "colsum_f32_noalloc: [" + std::to_string(rows) + "," + std::to_string(cols) + "] needs " +
                    std::to_string(need) + " bytes of scratch, the built-in array holds " +
                    std::to_string(kNoAllocScratchBytes) + "; use reduce_sum_keep_lastdim_f32_v0 with a workspace");
  }
  float* scratch = nullptr;
  const cudaError_t e = noalloc_scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(Status::Internal, std::string("colsum_f32_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
  }
  // Partials are fully rewritten for every (split, column) that the second pass reads, so nothing
  // left over from an earlier call needs clearing.
  const Status st = colsum_f32_direct(x, out, rows, cols, scratch, kNoAllocScratchBytes,
                                      reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(stream)));
  if (!ok(st)) return fail(st, std::string("colsum_f32_noalloc: launch failed: ") + status_to_string(st));
  return AICF_OK;
}
