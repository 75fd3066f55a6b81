// Layer norm over the last axis: forward (y, mean, rstd) and backward (dx, dgamma, dbeta).
//
// Contracts (same operand lists as the reference's layernorm launcher):
//   layernorm_fwd  inputs  [x (M,N), gamma (N), beta (N)]  or  [x]          attr: eps f32, schema 'LNEP', default 1e-5
//                  outputs [y (M,N), mean (M) f32, rstd (M) f32]
//   layernorm_bwd  inputs  [x, dy, gamma, mean, rstd] -> outputs [dx, dgamma (N) f32, dbeta (N) f32]
//                  inputs  [x, dy, mean, rstd]        -> outputs [dx]
//   x / y / dy / dx / gamma / beta share one dtype (f32, f16 or bf16); statistics and parameter gradients are f32.
//
// Forward is one HBM pass: a block owns a row at a time, holds it in registers, and has its next row in flight as a
// bulk asynchronous copy (the softmax kernels' pipeline). The variance is the mean of squared deviations from the
// row mean (both taken from registers), not E[x^2] - mean^2.
// Backward is one HBM pass as well: the same block keeps, per thread, running column sums of dy and dy * xhat for
// the columns it owns while it streams rows to produce dx; at the end every block writes its partial column sums to
// the workspace and a second small kernel adds the partials in block order (deterministic). x and dy are therefore
// read once, instead of once for dx and once more, column-strided, for the parameter gradients. Each block keeps a
// ring of up to four (x row, dy row) pairs in flight, spends two barriers per row, reads gamma once and requests a
// row's mean / rstd one iteration early.
// Rows that do not fit the register path (N not a multiple of the 16-byte packet, unaligned pointers, N beyond the
// per-thread element budget) take multi-pass kernels that accept anything.
#include <cstdlib>

#include "row_pipeline.cuh"

namespace aicf::cuda {

namespace {

using namespace rowk;

__device__ int g_ln_pipeline_status = 0;  // non-zero: a bounded wait of the row pipeline expired

// Two block-wide sums with two barriers. Every thread returns both totals. There is no barrier in front of the
// partial writes: the caller alternates between two `smem` areas from one call to the next, so a thread that is
// still reading the totals of call i cannot be overtaken by the partial writes of call i + 1 (those go to the
// other area), and call i + 2 is at least two barriers later. Work placed between the caller's shared-memory
// reads and this call is ordered before the first barrier for every thread.
constexpr int kSum2Floats = 2 * (kMaxWarps + 1);
__device__ __forceinline__ void block_sum2(float& a, float& b, float* smem /*[kSum2Floats]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  if (lane == 0) {
    smem[warp] = a;
    smem[kMaxWarps + 1 + warp] = b;
  }
  __syncthreads();
  if (warp == 0) {
    float ra = lane < nwarps ? smem[lane] : 0.0f;
    float rb = lane < nwarps ? smem[kMaxWarps + 1 + lane] : 0.0f;
    ra = warp_sum(ra);
    rb = warp_sum(rb);
    if (lane == 0) {
      smem[kMaxWarps] = ra;
      smem[2 * kMaxWarps + 1] = rb;
    }
  }
  __syncthreads();
  a = smem[kMaxWarps];
  b = smem[2 * kMaxWarps + 1];
}

template <typename T>
__device__ __forceinline__ Pack16<T> ld_param(const T* p, int64_t packet) {  // read-only path, stays in L1
  const int4 raw = __ldg(reinterpret_cast<const int4*>(p) + packet);
  Pack16<T> out;
  *reinterpret_cast<int4*>(&out) = raw;
  return out;
}

// ------------------------------------------------------------------ forward, row in registers
// kFull: the row is exactly kPackets packets for every thread of the block, so no packet needs a range check. The
// checks (a compare, a branch and a reconvergence point per packet and loop, and zero-fill of the unused registers)
// were a quarter of the instructions of the 16-bit kernels, which are bound by instruction issue.
template <typename T, int kPackets, bool kAffine, bool kFull>
__global__ void __launch_bounds__(1024)
    ln_fwd_regs_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                       float* __restrict__ mean, float* __restrict__ rstd, int64_t M, int64_t N, float eps) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  extern __shared__ __align__(16) uint8_t row_smem[];
  __shared__ float red[2][kMaxWarps + 1];
  __shared__ int wait_failed;
  using Idx = typename RowIdx<T>::type;
  const Idx np = static_cast<Idx>(N / kN);
  const uint32_t row_bytes = static_cast<uint32_t>(N * sizeof(T));
  const float inv_n = 1.0f / static_cast<float>(N);
  RowPipe pipe;
  pipe.init(row_smem, row_bytes, &wait_failed);
  int64_t row = blockIdx.x;
  if (row < M && threadIdx.x == 0) pipe.fetch(x + row * N, row_bytes);
  const PK* srow = reinterpret_cast<const PK*>(row_smem);
  for (; row < M; row += gridDim.x) {
    pipe.wait_row(&wait_failed);
    float f[kPackets][kN];
    float s = 0.0f;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        unpack16(srow[pi], f[q]);
#pragma unroll
        for (int e = 0; e < kN; ++e) s += f[q][e];
      } else {  // never read again (every later use sits behind the same range check); keeps the registers defined
#pragma unroll
        for (int e = 0; e < kN; ++e) f[q][e] = 0.0f;
      }
    }
    // Past the reduction's barriers the whole row is in registers everywhere and the buffer is free; a wait that
    // ran out is seen by all threads here.
    s = block_reduce_2b<false>(s, red[0]);
    if (wait_failed) {
      if (threadIdx.x == 0) atomicExch(&g_ln_pipeline_status, 1);
      break;
    }
    if (threadIdx.x == 0 && row + gridDim.x < M) {
      sm100::fence_generic_to_async_smem();
      pipe.fetch(x + (row + gridDim.x) * N, row_bytes);
    }
    const float mu = s * inv_n;
    float d2 = 0.0f;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
#pragma unroll
        for (int e = 0; e < kN; ++e) {
          f[q][e] -= mu;
          d2 = fmaf(f[q][e], f[q][e], d2);
        }
      }
    }
    d2 = block_reduce_2b<false>(d2, red[1]);
    const float rs = rsqrtf(d2 * inv_n + eps);
    if (threadIdx.x == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
    PK* yr = reinterpret_cast<PK*>(y + row * N);
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        PK o;
        float r[kN];
        if constexpr (kAffine) {
          float g[kN], b[kN];
          unpack16(ld_param(gamma, pi), g);
          unpack16(ld_param(beta, pi), b);
#pragma unroll
          for (int e = 0; e < kN; ++e) r[e] = fmaf(f[q][e] * rs, g[e], b[e]);
        } else {
#pragma unroll
          for (int e = 0; e < kN; ++e) r[e] = f[q][e] * rs;
        }
        pack16(o, r);
        st_stream(yr + pi, o);
      }
    }
  }
}

// Any N, any alignment: three reads of the row.
template <typename T>
__global__ void __launch_bounds__(256)
    ln_fwd_multipass_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                            T* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int64_t M, int64_t N,
                            float eps) {
  __shared__ float red[kMaxWarps + 1];
  const float inv_n = 1.0f / static_cast<float>(N);
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + row * N;
    T* yr = y + row * N;
    float s = 0.0f;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) s += Cvt<T>::to_f(xr[i]);
    const float mu = block_reduce<false>(s, red) * inv_n;
    float d2 = 0.0f;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
      const float d = Cvt<T>::to_f(xr[i]) - mu;
      d2 = fmaf(d, d, d2);
    }
    const float rs = rsqrtf(block_reduce<false>(d2, red) * inv_n + eps);
    if (threadIdx.x == 0) {
      mean[row] = mu;
      rstd[row] = rs;
    }
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
      float v = (Cvt<T>::to_f(xr[i]) - mu) * rs;
      if (gamma) v = fmaf(v, Cvt<T>::to_f(gamma[i]), Cvt<T>::to_f(beta[i]));
      yr[i] = Cvt<T>::from_f(v);
    }
  }
}

// ------------------------------------------------------------------ backward, rows in registers
// Dynamic shared memory: `stages` slots of [x row][dy row], then one mbarrier per slot. Slot i % stages holds the
// block's i-th row pair; a slot is refilled with the pair `stages` iterations ahead as soon as every thread has
// taken its part of the current pair into registers, so up to `stages` row pairs per block are in flight or
// waiting in shared memory while one is being worked on.
// partial: [gridDim.x][2][N] floats (dgamma partials, then dbeta partials), written only when kAffine.
template <typename T, int kPackets, bool kAffine, bool kFull>
__global__ void __launch_bounds__((kPackets * (16 / sizeof(T)) > 8) ? 512 : 1024)
    ln_bwd_regs_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                       const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx,
                       float* __restrict__ partial, int64_t M, int64_t N, int stages) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  extern __shared__ __align__(16) uint8_t row_smem[];
  __shared__ float red[2][kSum2Floats];
  __shared__ int wait_failed;
  using Idx = typename RowIdx<T>::type;
  const Idx np = static_cast<Idx>(N / kN);
  const uint32_t row_bytes = static_cast<uint32_t>(N * sizeof(T));
  const uint32_t slot_bytes = 2 * row_bytes;
  const float n_f = static_cast<float>(N), inv_n = 1.0f / n_f;
  const uint32_t buf0 = sm100::smem_addr(row_smem);
  const uint32_t bar0 = buf0 + static_cast<uint32_t>(stages) * slot_bytes;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) sm100::mbar_init(bar0 + 8u * s, 1);
    sm100::mbar_init_fence();
    wait_failed = 0;
  }
  __syncthreads();
  auto fetch2 = [&](int64_t r, int slot) {  // thread 0 only
    const uint32_t bar = bar0 + 8u * slot, buf = buf0 + static_cast<uint32_t>(slot) * slot_bytes;
    sm100::mbar_expect_tx(bar, slot_bytes);
    sm100::bulk_copy_g2s(buf, x + r * N, row_bytes, bar);
    sm100::bulk_copy_g2s(buf + row_bytes, dy + r * N, row_bytes, bar);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < stages; ++s) {
      const int64_t r = blockIdx.x + static_cast<int64_t>(s) * gridDim.x;
      if (r < M) fetch2(r, s);
    }
  float acc_g[kPackets][kN], acc_b[kPackets][kN];
#pragma unroll
  for (int q = 0; q < kPackets; ++q)
#pragma unroll
    for (int e = 0; e < kN; ++e) acc_g[q][e] = acc_b[q][e] = 0.0f;

  // This thread's columns never change: gamma is read once. The row statistics of the next row are requested one
  // iteration ahead, so their latency is not on the path between a row's arrival and its first arithmetic.
  float gam[kPackets][kN];
#pragma unroll
  for (int q = 0; q < kPackets; ++q) {
    const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
    PK pg;
    if (kAffine && (kFull || pi < np)) pg = ld_param(gamma, pi);
#pragma unroll
    for (int e = 0; e < kN; ++e) gam[q][e] = (kAffine && (kFull || pi < np)) ? Cvt<T>::to_f(pg.v[e]) : 1.0f;
  }
  int slot = 0, it = 0;
  uint32_t parity = 0;
  float mu_next = blockIdx.x < M ? __ldg(mean + blockIdx.x) : 0.0f;
  float rs_next = blockIdx.x < M ? __ldg(rstd + blockIdx.x) : 0.0f;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x, ++it) {
    const float mu = mu_next, rs = rs_next;
    if (row + gridDim.x < M) {
      mu_next = __ldg(mean + row + gridDim.x);
      rs_next = __ldg(rstd + row + gridDim.x);
    }
    // A wait that runs out is published through shared memory and acted on after the reduction's barriers, where
    // the whole block sees it: no barrier is spent on the wait itself.
    if (!sm100::mbar_wait_bounded(bar0 + 8u * slot, parity, kRowWaitBudgetNs)) wait_failed = 1;
    const PK* sx = reinterpret_cast<const PK*>(row_smem + static_cast<size_t>(slot) * slot_bytes);
    const PK* sdy = reinterpret_cast<const PK*>(row_smem + static_cast<size_t>(slot) * slot_bytes + row_bytes);
    float xh[kPackets][kN], g[kPackets][kN];
    float s1 = 0.0f, s2 = 0.0f;
    const float neg_mu_rs = -mu * rs;  // x-hat = x * rstd - mean * rstd: one fused multiply-add per element
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        const PK px = sx[pi], pd = sdy[pi];
#pragma unroll
        for (int e = 0; e < kN; ++e) {
          xh[q][e] = fmaf(Cvt<T>::to_f(px.v[e]), rs, neg_mu_rs);
          float d = Cvt<T>::to_f(pd.v[e]);
          if constexpr (kAffine) {
            acc_b[q][e] += d;
            acc_g[q][e] = fmaf(d, xh[q][e], acc_g[q][e]);
            d *= gam[q][e];
          }
          g[q][e] = d;
          s1 += d;
          s2 = fmaf(d, xh[q][e], s2);
        }
      } else {
#pragma unroll
        for (int e = 0; e < kN; ++e) xh[q][e] = g[q][e] = 0.0f;
      }
    }
    block_sum2(s1, s2, red[it & 1]);  // past its first barrier the pair is in registers everywhere: the slot is free
    if (wait_failed) {
      if (threadIdx.x == 0) atomicExch(&g_ln_pipeline_status, 1);
      break;
    }
    if (threadIdx.x == 0) {
      const int64_t ahead = row + static_cast<int64_t>(stages) * gridDim.x;
      if (ahead < M) {
        sm100::fence_generic_to_async_smem();
        fetch2(ahead, slot);
      }
    }
    // dx = (N g - s1 - x-hat s2) rstd / N, with the three row constants folded: two fused multiply-adds per element
    const float k = rs * inv_n;
    const float c_g = n_f * k, c_1 = -s1 * k, c_x = -s2 * k;
    PK* dxr = reinterpret_cast<PK*>(dx + row * N);
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        PK o;
        float r[kN];
#pragma unroll
        for (int e = 0; e < kN; ++e) r[e] = fmaf(g[q][e], c_g, fmaf(xh[q][e], c_x, c_1));
        pack16(o, r);
        st_stream(dxr + pi, o);
      }
    }
    if (++slot == stages) {
      slot = 0;
      parity ^= 1u;
    }
  }
  if constexpr (kAffine) {
    float* pg = partial + static_cast<int64_t>(blockIdx.x) * 2 * N;
    float* pb = pg + N;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
#pragma unroll
        for (int e = 0; e < kN; ++e) {
          pg[static_cast<int64_t>(pi) * kN + e] = acc_g[q][e];
          pb[static_cast<int64_t>(pi) * kN + e] = acc_b[q][e];
        }
      }
    }
  }
}

// dx for any N / alignment: two reads of x and dy.
template <typename T>
__global__ void __launch_bounds__(256)
    ln_bwd_dx_multipass_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                               const float* __restrict__ mean, const float* __restrict__ rstd, T* __restrict__ dx, int64_t M,
                               int64_t N) {
  __shared__ float red[2][kSum2Floats];
  int it = 0;
  const float n_f = static_cast<float>(N), inv_n = 1.0f / n_f;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + row * N;
    const T* dr = dy + row * N;
    T* o = dx + row * N;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.0f, s2 = 0.0f;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
      const float xh = (Cvt<T>::to_f(xr[i]) - mu) * rs;
      float d = Cvt<T>::to_f(dr[i]);
      if (gamma) d *= Cvt<T>::to_f(gamma[i]);
      s1 += d;
      s2 = fmaf(d, xh, s2);
    }
    block_sum2(s1, s2, red[it++ & 1]);
    const float k = rs * inv_n;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
      const float xh = (Cvt<T>::to_f(xr[i]) - mu) * rs;
      float d = Cvt<T>::to_f(dr[i]);
      if (gamma) d *= Cvt<T>::to_f(gamma[i]);
      o[i] = Cvt<T>::from_f((n_f * d - s1 - xh * s2) * k);
    }
  }
}

// Column partial sums for the multi-pass path: thread per column (coalesced along the row), blockIdx.y picks a
// slice of rows. partial: [gridDim.y][2][N].
template <typename T>
__global__ void __launch_bounds__(128)
    ln_bwd_colpartial_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ mean,
                             const float* __restrict__ rstd, float* __restrict__ partial, int64_t M, int64_t N) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float sg = 0.0f, sb = 0.0f;
  for (int64_t r = blockIdx.y; r < M; r += gridDim.y) {
    const float d = Cvt<T>::to_f(dy[r * N + c]);
    sb += d;
    sg = fmaf(d, (Cvt<T>::to_f(x[r * N + c]) - mean[r]) * rstd[r], sg);
  }
  float* p = partial + static_cast<int64_t>(blockIdx.y) * 2 * N;
  p[c] = sg;
  p[N + c] = sb;
}

// dgamma[c] = sum over slots of partial[slot][0][c], dbeta likewise. Block = 32 columns x 32 slot lanes: lane y adds
// slots y, y + 32, ... in order, then the 32 lane sums are added in lane order; the result does not depend on timing.
__global__ void __launch_bounds__(1024)
    ln_bwd_finish_kernel(const float* __restrict__ partial, float* __restrict__ dgamma, float* __restrict__ dbeta, int slots,
                         int64_t N) {
  __shared__ float lane_sum[32][33];
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 32 + threadIdx.x;  // over 2N: dgamma then dbeta
  float s = 0.0f;
  if (i < 2 * N)
    for (int b = threadIdx.y; b < slots; b += 32) s += partial[static_cast<int64_t>(b) * 2 * N + i];
  lane_sum[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < 2 * N) {
    float t = 0.0f;
#pragma unroll
    for (int y = 0; y < 32; ++y) t += lane_sum[y][threadIdx.x];
    if (i < N) dgamma[i] = t;
    else dbeta[i - N] = t;
  }
}

// ------------------------------------------------------------------ host side
float eps_of(const void* attr) {
  float eps = 1e-5f;
  read_attr_payload(attr, schema::kLayerNorm, /*allow_zero_schema=*/true, &eps, sizeof(eps));
  return eps;
}

bool vec_numel(const TensorDesc& t, DType dt, int64_t n) {  // contiguous vector of n elements of dtype dt
  if (t.dtype != dt || !t.contiguous) return false;
  int64_t have = 0;
  return positive_numel(t, 1, &have) && have == n;
}

template <DType kDt>
bool ln_fwd_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, int64_t* M, int64_t* N) {
  if (!in || !out || !(ni == 1 || ni == 3) || no != 3) return false;
  if (in[0].dtype != kDt || out[0].dtype != kDt || !in[0].contiguous || !out[0].contiguous) return false;
  if (!same_shape(in[0], out[0]) || !rows_cols_lastdim(in[0], M, N)) return false;
  if (!vec_numel(out[1], DType::kF32, *M) || !vec_numel(out[2], DType::kF32, *M)) return false;
  if (ni == 3 && (!vec_numel(in[1], kDt, *N) || !vec_numel(in[2], kDt, *N))) return false;
  return true;
}
template <DType kDt>
bool ln_fwd_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  int64_t M = 0, N = 0;
  return ln_fwd_check<kDt>(in, ni, out, no, &M, &N);
}

template <typename T, int kPackets, bool kAffine, bool kFull>
Status ln_fwd_go2(int threads, size_t smem, cudaStream_t stream, const T* x, const T* g, const T* b, T* y, float* mean,
                  float* rstd, int64_t M, int64_t N, float eps) {
  auto kernel = ln_fwd_regs_kernel<T, kPackets, kAffine, kFull>;
  if (!allow_smem(kernel, smem)) return Status::Internal;
  const int grid = streaming_grid(M, 1, row_blocks_per_sm(kernel, threads, smem));
  kernel<<<grid, threads, smem, stream>>>(x, g, b, y, mean, rstd, M, N, eps);
  return launch_status();
}
template <typename T, int kPackets>
Status ln_fwd_go(bool affine, int threads, size_t smem, cudaStream_t stream, const T* x, const T* g, const T* b, T* y,
                 float* mean, float* rstd, int64_t M, int64_t N, float eps) {
  const bool full = use_full_rows(N / Pack16<T>::kN == static_cast<int64_t>(threads) * kPackets, sizeof(T));
  if (affine)
    return full ? ln_fwd_go2<T, kPackets, true, true>(threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps)
                : ln_fwd_go2<T, kPackets, true, false>(threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps);
  return full ? ln_fwd_go2<T, kPackets, false, true>(threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps)
              : ln_fwd_go2<T, kPackets, false, false>(threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps);
}

template <DType kDt, typename T>
Status ln_fwd_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                     cudaStream_t stream) {
  int64_t M = 0, N = 0;
  if (!ln_fwd_check<kDt>(in, ni, out, no, &M, &N)) return Status::InvalidArgument;
  const bool affine = ni == 3;
  const T* x = static_cast<const T*>(in[0].data);
  const T* g = affine ? static_cast<const T*>(in[1].data) : nullptr;
  const T* b = affine ? static_cast<const T*>(in[2].data) : nullptr;
  T* y = static_cast<T*>(out[0].data);
  float* mean = static_cast<float*>(out[1].data);
  float* rstd = static_cast<float*>(out[2].data);
  const float eps = eps_of(attr);
  constexpr int kN = Pack16<T>::kN;
  constexpr int kMaxPk = sizeof(T) == 4 ? 8 : 4;
  const bool vec = (N % kN == 0) && aligned_to(x, 16) && aligned_to(y, 16) && (!affine || (aligned_to(g, 16) && aligned_to(b, 16)));
  const size_t smem = row_pipe_smem(N * static_cast<int64_t>(sizeof(T)));
  const RowCfg c = (vec && smem <= kMaxRowPipeSmem) ? pick_row_cfg(N / kN, kMaxPk) : RowCfg{};
  cudaGetLastError();
  if (c.packets == 0) {
    ln_fwd_multipass_kernel<T><<<streaming_grid(M, 1, 8), 256, 0, stream>>>(x, g, b, y, mean, rstd, M, N, eps);
    return launch_status();
  }
  switch (c.packets) {
    case 1: return ln_fwd_go<T, 1>(affine, c.threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps);
    case 2: return ln_fwd_go<T, 2>(affine, c.threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps);
    case 4: return ln_fwd_go<T, 4>(affine, c.threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps);
    default: return ln_fwd_go<T, kMaxPk>(affine, c.threads, smem, stream, x, g, b, y, mean, rstd, M, N, eps);
  }
}

// ---- backward
struct BwdGeom {
  int threads = 0, packets = 0;  // packets == 0: multi-pass path
  int grid = 0;                  // blocks of the register kernel (= partial slots on that path)
  int stages = 0;                // row pairs a block keeps in flight
  size_t smem = 0;
  int slices = 0;                // row slices (= partial slots) of the multi-pass path
};

// Register path: 8 row elements per thread (two fp32 packets or one 16-bit packet), so that x-hat, dy and the two
// column accumulators fit 64 registers and a 1024-thread block (N up to 8192) still launches; the shared memory
// an SM has left per resident block is then spent on prefetch depth. Wide 16-bit rows are the exception (below).
BwdGeom bwd_geom(int64_t M, int64_t N, size_t elem, bool vec_ok) {
  BwdGeom g;
  const int kn = static_cast<int>(16 / elem);
  // 16-bit rows of 512 elements and more take 16 elements per thread (two packets, ~110-120 registers, 512-thread
  // blocks at most): these kernels are bound by instruction issue, and the per-row overhead (barriers, shuffles, loop
  // control) is then spread over twice the elements. Fraction of the copy rate with 8 / 16 elements per thread, bf16:
  // 512 columns 0.57 / 0.77, 1024 0.67 / 0.79, 2048 0.69 / 0.81, 4096 0.78 / 0.92. Below 512 columns a warp would be left
  // with less than one packet pair per thread.
  // AICF_LN_BWD_WIDE_MIN (tuning, read once per process): the row length in packets from which the wide form is taken.
  static const int64_t wide_min = [] {
    const char* e = std::getenv("AICF_LN_BWD_WIDE_MIN");
    const long v = e ? std::atol(e) : 0;
    return static_cast<int64_t>(v > 0 ? v : 64);
  }();
  const bool wide = elem == 2 && N % kn == 0 && N / kn >= wide_min;
  const int max_packets = wide ? 2 : 8 / kn;
  const int64_t col_blocks = (N + 127) / 128;
  int64_t sl = (static_cast<int64_t>(sm_count()) * 8) / col_blocks;
  sl = sl < 1 ? 1 : sl;
  g.slices = static_cast<int>(sl < M ? sl : M);
  if (!vec_ok || N % kn != 0) return g;
  const int64_t np = N / kn;
  int threads = 32;
  while (threads < (wide ? 512 : 1024) && static_cast<int64_t>(threads) * max_packets < np) threads *= 2;
  const int64_t per = (np + threads - 1) / threads;
  if (per > max_packets) return g;
  const size_t slot = static_cast<size_t>(2 * N * elem);
  int resident = (wide ? 512 : 1024) / threads;  // blocks that fit the register file (64 or ~107 registers per thread)
  resident = resident > 32 ? 32 : resident;
  const size_t budget = (227 * 1024) / static_cast<size_t>(resident) - 1024;
  int stages = static_cast<int>((budget - 64) / slot);
  stages = stages > 4 ? 4 : stages;
  if (stages < 1) return g;
  g.threads = threads;
  g.packets = per <= 1 ? 1 : 2;
  g.stages = stages;
  g.smem = static_cast<size_t>(stages) * slot + 8 * static_cast<size_t>(stages) + 16;
  g.grid = streaming_grid(M, 1, resident);
  return g;
}

template <DType kDt>
bool ln_bwd_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, int64_t* M, int64_t* N) {
  if (!in || !out) return false;
  const bool affine = ni == 5 && no == 3, plain = ni == 4 && no == 1;
  if (!affine && !plain) return false;
  if (in[0].dtype != kDt || in[1].dtype != kDt || out[0].dtype != kDt) return false;
  if (!in[0].contiguous || !in[1].contiguous || !out[0].contiguous) return false;
  if (!same_shape(in[0], in[1]) || !same_shape(in[0], out[0]) || !rows_cols_lastdim(in[0], M, N)) return false;
  if (!vec_numel(in[affine ? 3 : 2], DType::kF32, *M) || !vec_numel(in[affine ? 4 : 3], DType::kF32, *M)) return false;
  if (affine && (!vec_numel(in[2], kDt, *N) || !vec_numel(out[1], DType::kF32, *N) || !vec_numel(out[2], DType::kF32, *N)))
    return false;
  return true;
}
template <DType kDt>
bool ln_bwd_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  int64_t M = 0, N = 0;
  return ln_bwd_check<kDt>(in, ni, out, no, &M, &N);
}

// Partial column sums of the affine form: [slots][2][N] floats, slots = the larger of the two paths' counts
// (which path runs depends on pointer alignment, unknown when the workspace is sized).
template <typename T>
size_t ln_bwd_workspace(const TensorDesc* in, int ni, const void*) {
  if (!in || ni != 5) return 0;
  int64_t M = 0, N = 0;
  if (!rows_cols_lastdim(in[0], &M, &N)) return 0;
  const BwdGeom a = bwd_geom(M, N, sizeof(T), true), b = bwd_geom(M, N, sizeof(T), false);
  const int slots = (a.packets ? a.grid : 0) > b.slices ? a.grid : b.slices;
  return static_cast<size_t>(slots) * 2 * static_cast<size_t>(N) * sizeof(float);
}

template <typename T, int kPackets, bool kAffine, bool kFull>
Status ln_bwd_go2(const BwdGeom& g, cudaStream_t stream, const T* x, const T* dy, const T* gamma, const float* mean,
                  const float* rstd, T* dx, float* partial, int64_t M, int64_t N) {
  auto kernel = ln_bwd_regs_kernel<T, kPackets, kAffine, kFull>;
  if (!allow_smem(kernel, g.smem)) return Status::Internal;
  kernel<<<g.grid, g.threads, g.smem, stream>>>(x, dy, gamma, mean, rstd, dx, partial, M, N, g.stages);
  return launch_status();
}
template <typename T, int kPackets>
Status ln_bwd_go(bool affine, const BwdGeom& g, cudaStream_t stream, const T* x, const T* dy, const T* gamma, const float* mean,
                 const float* rstd, T* dx, float* partial, int64_t M, int64_t N) {
  const bool full = use_full_rows(N / Pack16<T>::kN == static_cast<int64_t>(g.threads) * kPackets, sizeof(T));
  if (affine)
    return full ? ln_bwd_go2<T, kPackets, true, true>(g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N)
                : ln_bwd_go2<T, kPackets, true, false>(g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N);
  return full ? ln_bwd_go2<T, kPackets, false, true>(g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N)
              : ln_bwd_go2<T, kPackets, false, false>(g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N);
}

template <DType kDt, typename T>
Status ln_bwd_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void* ws, size_t ws_bytes,
                     cudaStream_t stream) {
  int64_t M = 0, N = 0;
  if (!ln_bwd_check<kDt>(in, ni, out, no, &M, &N)) return Status::InvalidArgument;
  const bool affine = ni == 5;
  const T* x = static_cast<const T*>(in[0].data);
  const T* dy = static_cast<const T*>(in[1].data);
  const T* gamma = affine ? static_cast<const T*>(in[2].data) : nullptr;
  const float* mean = static_cast<const float*>(in[affine ? 3 : 2].data);
  const float* rstd = static_cast<const float*>(in[affine ? 4 : 3].data);
  T* dx = static_cast<T*>(out[0].data);
  const bool vec = aligned_to(x, 16) && aligned_to(dy, 16) && aligned_to(dx, 16) && (!affine || aligned_to(gamma, 16));
  const BwdGeom g = bwd_geom(M, N, sizeof(T), vec);
  const int slots = g.packets ? g.grid : g.slices;
  float* partial = static_cast<float*>(ws);
  if (affine) {
    const size_t need = static_cast<size_t>(slots) * 2 * static_cast<size_t>(N) * sizeof(float);
    if (!ws || ws_bytes < need) return Status::InvalidArgument;
  }
  cudaGetLastError();
  Status st = Status::Ok;
  if (g.packets == 0) {
    ln_bwd_dx_multipass_kernel<T><<<streaming_grid(M, 1, 8), 256, 0, stream>>>(x, dy, gamma, mean, rstd, dx, M, N);
    st = launch_status();
    if (st == Status::Ok && affine) {
      const dim3 grid(static_cast<unsigned>((N + 127) / 128), static_cast<unsigned>(g.slices));
      ln_bwd_colpartial_kernel<T><<<grid, 128, 0, stream>>>(x, dy, mean, rstd, partial, M, N);
      st = launch_status();
    }
  } else {
    if (g.packets == 1) st = ln_bwd_go<T, 1>(affine, g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N);
    else if constexpr (sizeof(T) == 4) st = ln_bwd_go<T, 2>(affine, g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N);
    else st = ln_bwd_go<T, 2>(affine, g, stream, x, dy, gamma, mean, rstd, dx, partial, M, N);
  }
  if (st != Status::Ok || !affine) return st;
  ln_bwd_finish_kernel<<<static_cast<unsigned>((2 * N + 31) / 32), dim3(32, 32), 0, stream>>>(
      partial, static_cast<float*>(out[1].data), static_cast<float*>(out[2].data), slots, N);
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
  v.expected_attr_schema_id = 0;  // 'LNEP' carries eps; schema 0 (no attrs) means the default eps
  v.launch = l;
  v.supported = s;
  v.query_workspace = w;
  return v;
}

}  // namespace

// Reads (optionally clears) the status word of the layer-norm kernels' bounded waits. Synchronises the device.
int layernorm_pipeline_status(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_ln_pipeline_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (clear && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_ln_pipeline_status, &zero, sizeof(int));
  }
  return v;
}

KernelVariant make_layernorm_fwd_f32_variant() { return make("layernorm_fwd_f32_sm100", ln_fwd_launch<DType::kF32, float>, ln_fwd_supported<DType::kF32>, no_workspace); }
KernelVariant make_layernorm_fwd_f16_variant() { return make("layernorm_fwd_f16_sm100", ln_fwd_launch<DType::kF16, __half>, ln_fwd_supported<DType::kF16>, no_workspace); }
KernelVariant make_layernorm_fwd_bf16_variant() { return make("layernorm_fwd_bf16_sm100", ln_fwd_launch<DType::kBF16, __nv_bfloat16>, ln_fwd_supported<DType::kBF16>, no_workspace); }
KernelVariant make_layernorm_bwd_f32_variant() { return make("layernorm_bwd_f32_sm100", ln_bwd_launch<DType::kF32, float>, ln_bwd_supported<DType::kF32>, ln_bwd_workspace<float>); }
KernelVariant make_layernorm_bwd_f16_variant() { return make("layernorm_bwd_f16_sm100", ln_bwd_launch<DType::kF16, __half>, ln_bwd_supported<DType::kF16>, ln_bwd_workspace<__half>); }
KernelVariant make_layernorm_bwd_bf16_variant() { return make("layernorm_bwd_bf16_sm100", ln_bwd_launch<DType::kBF16, __nv_bfloat16>, ln_bwd_supported<DType::kBF16>, ln_bwd_workspace<__nv_bfloat16>); }

}  // namespace aicf::cuda
