// Row softmax and fused softmax cross-entropy (loss rows + gradient + argmax) over the last axis.
//
// Single HBM pass: a block owns one row at a time and keeps it in registers (kPackets 16-byte
// packets per thread), so the row is read once and the result written once. While a row is being
// reduced, exponentiated and stored from registers, the block's NEXT row is already on its way into
// shared memory as one bulk asynchronous copy (cp.async.bulk + mbarrier), so every SM always has a
// row-sized read in flight and the load / reduce / store phases of a block overlap with each other.
// Row max / sum are warp-shuffle reductions joined through shared memory in a fixed order, hence
// deterministic.
// Two more single-pass forms beside these persistent, pipelined kernels: softmax rows that 128 threads or
// fewer hold at exactly four packets each go one row per block straight from global memory into
// registers (softmax_direct_kernel), and fp32 cross-entropy rows too long for one block's registers
// (32768 to 65536 columns) go one row per thread-block cluster (softmax_ce_cluster_kernel).
// Everything else (softmax rows wider than 32768 elements, rows that are not 16-byte aligned) takes a
// three-read fallback kernel.
#include <cstdlib>

#include "row_pipeline.cuh"

namespace aicf::cuda {

namespace {

using namespace rowk;

// exp(v - mx) for v <= mx: a subtraction, a multiply by log2(e) and one MUFU.EX2. Relative error <= |v - mx| * 2^-24
// + 2^-22, i.e. below 1e-5 for every argument whose result is not already flushed to zero; the accurate expf costs
// ~20 instructions per element, which for a 32000-wide row is more time than its HBM traffic. The subtraction comes
// first on purpose: the row maximum itself then gives exp2(0) = 1 exactly, which a loss of the order of 1e-6 (a
// confident, correct prediction: sum = 1 + a few e-6) depends on. Folding the shift into one fused multiply-add
// (2^(v * log2(e) - mx * log2(e))) saves an instruction but puts the rounding of mx * log2(e), up to 1e-6, into
// log(sum).
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float exp2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float exp_shifted(float v, float mx) { return exp2_approx((v - mx) * kLog2e); }

struct ArgMax {
  float v;
  int idx;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {  // larger value wins, ties -> lower index
  if (b.v > a.v || (b.v == a.v && b.idx < a.idx)) return b;
  return a;
}
__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.idx = __shfl_xor_sync(0xffffffffu, a.idx, o);
    a = better(a, b);
  }
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, float* sv /*[kMaxWarps + 1]*/, int* si /*[kMaxWarps + 1]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  a = warp_argmax(a);
  __syncthreads();
  if (lane == 0) {
    sv[warp] = a.v;
    si[warp] = a.idx;
  }
  __syncthreads();
  if (warp == 0) {
    ArgMax r{lane < nwarps ? sv[lane] : -INFINITY, lane < nwarps ? si[lane] : 0x7fffffff};
    r = warp_argmax(r);
    if (lane == 0) {
      sv[kMaxWarps] = r.v;
      si[kMaxWarps] = r.idx;
    }
  }
  __syncthreads();
  return ArgMax{sv[kMaxWarps], si[kMaxWarps]};
}

__device__ int g_row_pipeline_status = 0;  // non-zero: a bounded wait of the row pipeline expired

// Block-wide sum of `s` and minimum of `idx` in one trip through shared memory. kLeadingBarrier as in block_reduce
// (areas possibly still being read by the previous call) against block_reduce_2b (caller alternates areas).
struct SumMin {
  float sum;
  int idx;
};
template <bool kLeadingBarrier>
__device__ __forceinline__ SumMin block_sum_min(float s, int idx, float* sv /*[kMaxWarps + 1]*/, int* si /*[kMaxWarps + 1]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  s = warp_sum(s);
  idx = __reduce_min_sync(0xffffffffu, idx);
  if (kLeadingBarrier) __syncthreads();
  if (lane == 0) {
    sv[warp] = s;
    si[warp] = idx;
  }
  __syncthreads();
  if (warp == 0) {
    float r = lane < nwarps ? sv[lane] : 0.0f;
    int j = lane < nwarps ? si[lane] : 0x7fffffff;
    r = warp_sum(r);
    j = __reduce_min_sync(0xffffffffu, j);
    if (lane == 0) {
      sv[kMaxWarps] = r;
      si[kMaxWarps] = j;
    }
  }
  __syncthreads();
  return SumMin{sv[kMaxWarps], si[kMaxWarps]};
}

// ------------------------------------------------------------------ softmax, row in registers
// kFull: the row is exactly kPackets packets for every thread, so no packet needs a range check (a compare, a branch and a
// reconvergence point per packet and loop otherwise: a sizeable share of the instructions of the 16-bit kernels).
template <typename T, int kPackets, bool kFull>
__global__ void __launch_bounds__(1024) softmax_regs_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t M,
                                                           int64_t N) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  extern __shared__ __align__(16) uint8_t row_smem[];
  __shared__ float red[2][kMaxWarps + 1];
  __shared__ int wait_failed;
  using Idx = typename RowIdx<T>::type;
  const Idx np = static_cast<Idx>(N / kN);  // N % kN == 0 on this path
  const uint32_t row_bytes = static_cast<uint32_t>(N * sizeof(T));
  RowPipe pipe;
  pipe.init(row_smem, row_bytes, &wait_failed);
  int64_t row = blockIdx.x;
  if (row < M && threadIdx.x == 0) pipe.fetch(x + row * N, row_bytes);
  const PK* srow = reinterpret_cast<const PK*>(row_smem);
  for (; row < M; row += gridDim.x) {
    pipe.wait_row(&wait_failed);
    PK* yr = reinterpret_cast<PK*>(y + row * N);
    float f[kPackets][kN];
    float mx = -INFINITY;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        unpack16(srow[pi], f[q]);
#pragma unroll
        for (int e = 0; e < kN; ++e) mx = fmaxf(mx, f[q][e]);
      } else {
#pragma unroll
        for (int e = 0; e < kN; ++e) f[q][e] = -INFINITY;
      }
    }
    // Past the reduction's barriers every thread has copied its part of the row out of shared memory, so thread 0
    // may let the next row overwrite the buffer; a wait that ran out is seen by all threads here.
    mx = block_reduce_2b<true>(mx, red[0]);
    if (wait_failed) {
      if (threadIdx.x == 0) atomicExch(&g_row_pipeline_status, 1);
      break;
    }
    if (threadIdx.x == 0 && row + gridDim.x < M) {
      sm100::fence_generic_to_async_smem();
      pipe.fetch(x + (row + gridDim.x) * N, row_bytes);
    }
    float sum = 0.0f;
#pragma unroll
    for (int q = 0; q < kPackets; ++q)
#pragma unroll
      for (int e = 0; e < kN; ++e) {
        f[q][e] = exp_shifted(f[q][e], mx);  // exp(-inf) == 0 for the padding
        sum += f[q][e];
      }
    sum = block_reduce_2b<false>(sum, red[1]);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        PK o;
        float r[kN];
#pragma unroll
        for (int e = 0; e < kN; ++e) r[e] = f[q][e] * inv;
        pack16(o, r);
        st_stream(yr + pi, o);
      }
    }
  }
}

// One row per block, straight from global memory into registers: no staging buffer, no barrier object, nothing that
// outlives the row. The grid has a block per row (grid-stride past the launch limit), so an SM always has several
// rows at different stages and the hardware's block scheduler does the load balancing.
template <typename T, int kPackets, bool kFull>
__global__ void __launch_bounds__(1024) softmax_direct_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t M,
                                                             int64_t N) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  __shared__ float red[2][kMaxWarps + 1];
  using Idx = typename RowIdx<T>::type;
  const Idx np = static_cast<Idx>(N / kN);
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const PK* xr = reinterpret_cast<const PK*>(x + row * N);
    PK* yr = reinterpret_cast<PK*>(y + row * N);
    PK raw[kPackets];
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) raw[q] = ld_stream(xr + pi);
    }
    float f[kPackets][kN];
    float mx = -INFINITY;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        unpack16(raw[q], f[q]);
#pragma unroll
        for (int e = 0; e < kN; ++e) mx = fmaxf(mx, f[q][e]);
      } else {
#pragma unroll
        for (int e = 0; e < kN; ++e) f[q][e] = -INFINITY;
      }
    }
    mx = block_reduce_2b<true>(mx, red[0]);
    float sum = 0.0f;
#pragma unroll
    for (int q = 0; q < kPackets; ++q)
#pragma unroll
      for (int e = 0; e < kN; ++e) {
        f[q][e] = exp_shifted(f[q][e], mx);
        sum += f[q][e];
      }
    sum = block_reduce_2b<false>(sum, red[1]);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        PK o;
        float r[kN];
#pragma unroll
        for (int e = 0; e < kN; ++e) r[e] = f[q][e] * inv;
        pack16(o, r);
        st_stream(yr + pi, o);
      }
    }
  }
}

// Fallback: any N, any alignment; reads the row three times.
template <typename T>
__global__ void __launch_bounds__(256) softmax_multipass_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t M,
                                                               int64_t N) {
  __shared__ float red[kMaxWarps + 1];
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + row * N;
    T* yr = y + row * N;
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) mx = fmaxf(mx, Cvt<T>::to_f(xr[i]));
    mx = block_reduce<true>(mx, red);
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) sum += expf(Cvt<T>::to_f(xr[i]) - mx);
    sum = block_reduce<false>(sum, red);
    const float inv = 1.0f / sum;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x) yr[i] = Cvt<T>::from_f(expf(Cvt<T>::to_f(xr[i]) - mx) * inv);
  }
}

template <typename T>
Status softmax_run(const T* x, T* y, int64_t M, int64_t N, cudaStream_t stream) {
  constexpr int kN = Pack16<T>::kN;
  constexpr int kMaxPk = sizeof(T) == 4 ? 8 : 4;
  const bool vec = (N % kN == 0) && aligned_to(x, 16) && aligned_to(y, 16);
  const size_t smem = row_pipe_smem(N * static_cast<int64_t>(sizeof(T)));
  const RowCfg c = (vec && smem <= kMaxRowPipeSmem) ? pick_row_cfg(N / kN, kMaxPk) : RowCfg{};
  cudaGetLastError();
  if (c.packets == 0) {
    softmax_multipass_kernel<T><<<streaming_grid(M, 1, 8), 256, 0, stream>>>(x, y, M, N);
    return launch_status();
  }
  bool ok_attr = true;
  const bool full = use_full_rows(N / kN == static_cast<int64_t>(c.threads) * c.packets, sizeof(T));
  // Rows that small blocks (up to 128 threads) hold at four packets per thread go one row per block, straight into
  // registers, when the row fills those packets exactly (1536 columns of bf16, three packets of four used: 5422 direct,
  // 5934 pipelined); longer rows keep the persistent blocks with the prefetched row buffer, shorter ones too. GB/s, direct
  // against pipelined: f32 1024 columns 6873 / 6142, 2048 6741 / 6483, 4096 (256 threads) 6471 / 6624, 8192 5880 /
  // 6405, 256 5636 / 6058; bf16 1024 6540 / 5584, 2048 6496 / 6275, 4096 (128 threads) 6522 / 6475, 8192 6041 / 6227.
  // AICF_SOFTMAX_DIRECT=0|1 (tuning, read once per process) forces one or the other.
  static const int direct_override = [] {
    const char* e = std::getenv("AICF_SOFTMAX_DIRECT");
    return (e == nullptr || e[0] == 0) ? -1 : (e[0] == '0' ? 0 : 1);
  }();
  const bool exact_fit = N / kN == static_cast<int64_t>(c.threads) * c.packets;
  const bool direct = direct_override >= 0 ? direct_override != 0 : (c.threads <= 128 && c.packets >= 4 && exact_fit);
  if (direct) {
    const int grid = streaming_grid(M, 1, kStreamBlocksPerSm);
#define AICF_SM_DIRECT(PK, FULL) softmax_direct_kernel<T, PK, FULL><<<grid, c.threads, 0, stream>>>(x, y, M, N)
#define AICF_SM_DIRECT_F(PK)            \
  if (full) { AICF_SM_DIRECT(PK, true); } \
  else { AICF_SM_DIRECT(PK, false); }
    switch (c.packets) {
      case 1: AICF_SM_DIRECT_F(1); break;
      case 2: AICF_SM_DIRECT_F(2); break;
      case 4: AICF_SM_DIRECT_F(4); break;
      default: AICF_SM_DIRECT_F(kMaxPk); break;
    }
#undef AICF_SM_DIRECT_F
#undef AICF_SM_DIRECT
    return launch_status();
  }
  const size_t smem_launch = row_smem_capped_residency(smem, c.threads);  // the grid is still sized from `smem`
#define AICF_SM_LAUNCH_F(PK, FULL)                                                                                 \
  if ((ok_attr = allow_smem(softmax_regs_kernel<T, PK, FULL>, smem_launch)))                                       \
    softmax_regs_kernel<T, PK, FULL>                                                                               \
        <<<streaming_grid(M, 1, row_blocks_per_sm(softmax_regs_kernel<T, PK, FULL>, c.threads, smem)), c.threads, \
           smem_launch, stream>>>(x, y, M, N)
#define AICF_SM_LAUNCH(PK)                     \
  if (full) { AICF_SM_LAUNCH_F(PK, true); }    \
  else { AICF_SM_LAUNCH_F(PK, false); }
  switch (c.packets) {
    case 1: AICF_SM_LAUNCH(1); break;
    case 2: AICF_SM_LAUNCH(2); break;
    case 4: AICF_SM_LAUNCH(4); break;
    default: AICF_SM_LAUNCH(kMaxPk); break;
  }
#undef AICF_SM_LAUNCH
#undef AICF_SM_LAUNCH_F
  if (!ok_attr) {
    cudaGetLastError();
    return Status::Internal;
  }
  return launch_status();
}

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

template <DType kDt>
bool softmax_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != kDt || out[0].dtype != kDt) return false;
  if (!in[0].contiguous || !out[0].contiguous || !same_shape(in[0], out[0])) return false;
  int64_t M = 0, N = 0;
  return rows_cols_any(in[0], &M, &N);
}
template <DType kDt>
bool softmax_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return softmax_check<kDt>(in, ni, out, no);
}
template <DType kDt, typename T>
Status softmax_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t,
                      cudaStream_t stream) {
  if (!softmax_check<kDt>(in, ni, out, no)) return Status::InvalidArgument;
  int64_t M = 0, N = 0;
  rows_cols_any(in[0], &M, &N);
  return softmax_run<T>(static_cast<const T*>(in[0].data), static_cast<T*>(out[0].data), M, N, stream);
}

// ------------------------------------------------------------------ softmax cross-entropy
// inputs  [logits (B,C) f32|bf16|f16, labels (B,) i32]
// outputs [dlogits (B,C) same dtype, loss_row (B,) f32, argmax (B,) i32]   (argmax optional)
//   loss_row = logsumexp(z) - z[label];  dlogits = (softmax(z) - onehot(label)) * scale
// scale: 'SMCE' <f>, default 1/B. A label outside [0,C) contributes no one-hot term and a zero loss.
// kLockstep: the wait for the row ends in a barrier and the reductions keep their leading barrier (an alternative
// form kept for tuning, see the launcher; the two-barrier form is what runs).
// Per element the loops only take a maximum, an exponential and a product: the arg-max index is looked up afterwards
// by the few threads that hold the row maximum and reduced together with the sum, and the one-hot term is patched in
// by the one thread that owns the label's column.
template <typename T, int kPackets, bool kLockstep, bool kFull, bool kEarlyRefill>
__global__ void __launch_bounds__(1024)
    softmax_ce_regs_kernel(const T* __restrict__ z, const int32_t* __restrict__ labels, T* __restrict__ dz,
                           float* __restrict__ loss_row, int32_t* __restrict__ argmax_out, int64_t B, int64_t C,
                           float scale) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  extern __shared__ __align__(16) uint8_t row_smem[];
  __shared__ float red[2][kMaxWarps + 1];
  __shared__ int wait_failed;
  __shared__ int redi[kMaxWarps + 1];
  using Idx = typename RowIdx<T>::type;
  const Idx np = static_cast<Idx>(C / kN);
  const uint32_t row_bytes = static_cast<uint32_t>(C * sizeof(T));
  RowPipe pipe;
  pipe.init(row_smem, row_bytes, &wait_failed);
  int64_t row = blockIdx.x;
  if (row < B && threadIdx.x == 0) pipe.fetch(z + row * C, row_bytes);
  const PK* srow = reinterpret_cast<const PK*>(row_smem);
  for (; row < B; row += gridDim.x) {
    if constexpr (kLockstep) {
      if (!pipe.arrived(&g_row_pipeline_status)) break;
    } else {
      pipe.wait_row(&wait_failed);
    }
    PK* dr = reinterpret_cast<PK*>(dz + row * C);
    const int label = labels[row];
    const bool label_ok = label >= 0 && label < C;
    // The thread whose packets hold column `label` patches the one-hot term after its stores (same thread, same
    // address: ordered), so the element loops carry no per-element column compare. It and thread 0 (loss) read the
    // label's logit while the row is still in shared memory.
    const int owner = label_ok ? static_cast<int>((label / kN) % static_cast<int>(blockDim.x)) : -1;
    float z_label = 0.0f;
    if (label_ok && (threadIdx.x == 0 || static_cast<int>(threadIdx.x) == owner))
      z_label = Cvt<T>::to_f(reinterpret_cast<const T*>(row_smem)[label]);
    // With kEarlyRefill (one block per SM: nobody else keeps the SM's loads going) the row is first only taken out of
    // shared memory, a barrier of its own follows at once and the next row is requested before any arithmetic, instead
    // of after the maximum's reduction: the time an SM has no load in flight shrinks from the copy, the maximum and its
    // two barriers to the copy and one barrier.
    constexpr bool early = !kLockstep && kEarlyRefill;
    auto refill = [&]() {  // after a block-wide barrier: every thread holds its packets, a failed wait is seen by all
      if (threadIdx.x == 0 && row + gridDim.x < B) {
        sm100::fence_generic_to_async_smem();
        pipe.fetch(z + (row + gridDim.x) * C, row_bytes);
      }
    };
    float f[kPackets][kN];
    float tmax = -INFINITY;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        unpack16(srow[pi], f[q]);
        if constexpr (!early) {
#pragma unroll
          for (int e = 0; e < kN; ++e) tmax = fmaxf(tmax, f[q][e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < kN; ++e) f[q][e] = -INFINITY;
      }
    }
    if constexpr (early) {
      __syncthreads();
      if (wait_failed) {
        if (threadIdx.x == 0) atomicExch(&g_row_pipeline_status, 1);
        break;
      }
      refill();
#pragma unroll
      for (int q = 0; q < kPackets; ++q)
#pragma unroll
        for (int e = 0; e < kN; ++e) tmax = fmaxf(tmax, f[q][e]);  // the padding is -inf
    }
    const float mx = kLockstep ? block_reduce<true>(tmax, red[0]) : block_reduce_2b<true>(tmax, red[0]);
    if (!early) {
      if (wait_failed) {
        if (threadIdx.x == 0) atomicExch(&g_row_pipeline_status, 1);
        break;
      }
      refill();
    }
    // arg-max: only the (few) threads that hold the row maximum look for its lowest column among their elements;
    // the block-wide minimum of those candidates rides along with the sum reduction below
    int cand = 0x7fffffff;
    if (tmax == mx) {
#pragma unroll
      for (int q = kPackets - 1; q >= 0; --q) {
        const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
        if (kFull || pi < np) {
#pragma unroll
          for (int e = kN - 1; e >= 0; --e)
            if (f[q][e] == mx) cand = static_cast<int>(pi) * kN + e;  // descending order: the lowest column stays
        }
      }
    }
    float sum = 0.0f;
#pragma unroll
    for (int q = 0; q < kPackets; ++q)
#pragma unroll
      for (int e = 0; e < kN; ++e) {
        f[q][e] = exp_shifted(f[q][e], mx);
        sum += f[q][e];
      }
    const SumMin sm = block_sum_min<kLockstep>(sum, cand, red[1], redi);
    sum = sm.sum;
    const float k = scale / sum;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const Idx pi = static_cast<Idx>(threadIdx.x) + static_cast<Idx>(q) * static_cast<Idx>(blockDim.x);
      if (kFull || pi < np) {
        PK o;
        float r[kN];
#pragma unroll
        for (int e = 0; e < kN; ++e) r[e] = f[q][e] * k;
        pack16(o, r);
        st_stream(dr + pi, o);
      }
    }
    if (static_cast<int>(threadIdx.x) == owner) {
      const float g = exp_shifted(z_label, mx) * k - scale;  // the same bits the loop above produced, minus the one-hot term
      dz[row * C + label] = Cvt<T>::from_f(g);
    }
    if (threadIdx.x == 0) {
      loss_row[row] = label_ok ? (logf(sum) + mx - z_label) : 0.0f;
      if (argmax_out) argmax_out[row] = sm.idx;
    }
  }
}

// ---- very long rows: one row per thread-block cluster ----------------------------------------------------------------
// A row that no single block can hold in registers is split over the 2, 4 or 8 CTAs of a cluster: each CTA keeps a
// contiguous slice of the row in registers, loaded straight from global memory, and the CTAs exchange the two per-row
// scalars (maximum, then sum and arg-max candidate) through each other's shared memory between cluster barriers. The row
// is still read once and written once. Partial sums are added in rank order, so the result does not depend on timing.
constexpr int kClusterThreads = 256;
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_index() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// Every thread of every CTA of the cluster; orders shared-memory writes before it against peers' reads after it.
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The 4-byte word at `local`'s offset in the shared memory of CTA `rank` of this cluster.
template <typename V>
__device__ __forceinline__ V ld_peer_shared(const V* local, uint32_t rank) {
  static_assert(sizeof(V) == 4, "4-byte words only");
  const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote, bits;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(bits) : "r"(remote) : "memory");
  V v;
  memcpy(&v, &bits, 4);
  return v;
}

template <typename T, int kPackets>
__global__ void __launch_bounds__(kClusterThreads, 4)  // four CTAs per SM: 64 registers
    softmax_ce_cluster_kernel(const T* __restrict__ z, const int32_t* __restrict__ labels, T* __restrict__ dz,
                              float* __restrict__ loss_row, int32_t* __restrict__ argmax_out, int64_t B, int64_t C,
                              float scale, int slice /* packets per CTA */) {
  using PK = Pack16<T>;
  constexpr int kN = PK::kN;
  __shared__ float red[2][kMaxWarps + 1];
  __shared__ int redi[kMaxWarps + 1];
  __shared__ float x_max, x_sum;  // this CTA's share of the row's maximum and sum, read by its peers
  __shared__ int x_cand;          // and its lowest column holding the row maximum
  const uint32_t rank = cluster_rank(), nranks = cluster_size();
  const int np = static_cast<int>(C / kN);
  const int p0 = static_cast<int>(rank) * slice;               // first packet of this CTA's slice
  const int pn = np - p0 < slice ? (np - p0 > 0 ? np - p0 : 0) : slice;  // packets in it
  for (int64_t row = cluster_index(); row < B; row += cluster_count()) {
    const PK* zr = reinterpret_cast<const PK*>(z + row * C) + p0;
    PK* dr = reinterpret_cast<PK*>(dz + row * C) + p0;
    const int label = labels[row];
    const bool label_ok = label >= 0 && label < C;
    // the one thread of the cluster whose packets hold column `label`: it patches the one-hot term and writes the loss
    const int lp = label_ok ? label / kN - p0 : -1;
    const bool owner = lp >= 0 && lp < pn && lp % kClusterThreads == static_cast<int>(threadIdx.x);
    const float z_label = owner ? Cvt<T>::to_f(z[row * C + label]) : 0.0f;
    PK raw[kPackets];
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const int pi = static_cast<int>(threadIdx.x) + q * kClusterThreads;
      if (pi < pn) raw[q] = ld_stream(zr + pi);
    }
    float f[kPackets][kN];
    float tmax = -INFINITY;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const int pi = static_cast<int>(threadIdx.x) + q * kClusterThreads;
      if (pi < pn) {
        unpack16(raw[q], f[q]);
#pragma unroll
        for (int e = 0; e < kN; ++e) tmax = fmaxf(tmax, f[q][e]);
      } else {
#pragma unroll
        for (int e = 0; e < kN; ++e) f[q][e] = -INFINITY;
      }
    }
    const float local_max = block_reduce_2b<true>(tmax, red[0]);
    if (threadIdx.x == 0) x_max = local_max;
    cluster_barrier();
    float mx = -INFINITY;
    for (uint32_t r = 0; r < nranks; ++r) mx = fmaxf(mx, ld_peer_shared(&x_max, r));
    int cand = 0x7fffffff;
    if (tmax == mx) {
#pragma unroll
      for (int q = kPackets - 1; q >= 0; --q) {
        const int pi = static_cast<int>(threadIdx.x) + q * kClusterThreads;
        if (pi < pn) {
#pragma unroll
          for (int e = kN - 1; e >= 0; --e)
            if (f[q][e] == mx) cand = (p0 + pi) * kN + e;  // descending order: the lowest column stays
        }
      }
    }
    float sum = 0.0f;
#pragma unroll
    for (int q = 0; q < kPackets; ++q)
#pragma unroll
      for (int e = 0; e < kN; ++e) {
        f[q][e] = exp_shifted(f[q][e], mx);  // exp(-inf) == 0 for the padding
        sum += f[q][e];
      }
    const SumMin local = block_sum_min<false>(sum, cand, red[1], redi);
    if (threadIdx.x == 0) {
      x_sum = local.sum;
      x_cand = local.idx;
    }
    cluster_barrier();  // every CTA is past its reads of x_max, too: the next row may overwrite it
    float total = 0.0f;
    int best = 0x7fffffff;
    for (uint32_t r = 0; r < nranks; ++r) {
      total += ld_peer_shared(&x_sum, r);
      const int c = ld_peer_shared(&x_cand, r);
      best = c < best ? c : best;
    }
    const float k = scale / total;
#pragma unroll
    for (int q = 0; q < kPackets; ++q) {
      const int pi = static_cast<int>(threadIdx.x) + q * kClusterThreads;
      if (pi < pn) {
        PK o;
        float r[kN];
#pragma unroll
        for (int e = 0; e < kN; ++e) r[e] = f[q][e] * k;
        pack16(o, r);
        st_stream(dr + pi, o);
      }
    }
    if (owner) {
      const float g = exp_shifted(z_label, mx) * k - scale;  // the same bits the loop above produced, minus the one-hot term
      dz[row * C + label] = Cvt<T>::from_f(g);
      loss_row[row] = logf(total) + mx - z_label;
    }
    if (rank == 0 && threadIdx.x == 0) {
      if (!label_ok) loss_row[row] = 0.0f;
      if (argmax_out) argmax_out[row] = best;
    }
    // x_sum / x_cand of this row are read before a peer arrives at the next row's first cluster barrier, and they are
    // next written after that barrier: no third barrier needed inside the loop
  }
  cluster_barrier();  // nobody leaves while a peer may still be reading its shared memory
}

template <typename T>
__global__ void __launch_bounds__(256)
    softmax_ce_multipass_kernel(const T* __restrict__ z, const int32_t* __restrict__ labels, T* __restrict__ dz,
                                float* __restrict__ loss_row, int32_t* __restrict__ argmax_out, int64_t B, int64_t C,
                                float scale) {
  __shared__ float red[kMaxWarps + 1];
  __shared__ int redi[kMaxWarps + 1];
  for (int64_t row = blockIdx.x; row < B; row += gridDim.x) {
    const T* zr = z + row * C;
    T* dr = dz + row * C;
    const int label = labels[row];
    ArgMax am{-INFINITY, 0x7fffffff};
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) {
      const float v = Cvt<T>::to_f(zr[i]);
      if (v > am.v) {
        am.v = v;
        am.idx = static_cast<int>(i);
      }
    }
    am = block_argmax(am, red, redi);
    const float mx = am.v;
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) sum += expf(Cvt<T>::to_f(zr[i]) - mx);
    sum = block_reduce<false>(sum, red);
    const float k = scale / sum;
    for (int64_t i = threadIdx.x; i < C; i += blockDim.x) {
      float g = expf(Cvt<T>::to_f(zr[i]) - mx) * k;
      if (i == label) g -= scale;
      dr[i] = Cvt<T>::from_f(g);
    }
    if (threadIdx.x == 0) {
      const bool label_ok = label >= 0 && label < C;
      loss_row[row] = label_ok ? (logf(sum) + mx - Cvt<T>::to_f(zr[label_ok ? label : 0])) : 0.0f;
      if (argmax_out) argmax_out[row] = am.idx;
    }
    __syncthreads();
  }
}

template <DType kDt>
bool softmax_ce_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 2 || (no != 2 && no != 3)) return false;
  const TensorDesc &Z = in[0], &L = in[1], &D = out[0], &Lo = out[1];
  if (Z.dtype != kDt || D.dtype != kDt || Z.rank() != 2 || !Z.contiguous || !D.contiguous || !same_shape(Z, D))
    return false;
  if (Z.shape[0] <= 0 || Z.shape[1] <= 0 || Z.shape[1] > 0x7fffffff) return false;
  if (L.dtype != DType::kI32 || L.rank() != 1 || !L.contiguous || L.shape[0] != Z.shape[0]) return false;
  if (Lo.dtype != DType::kF32 || Lo.rank() != 1 || !Lo.contiguous || Lo.shape[0] != Z.shape[0]) return false;
  if (no == 3) {
    const TensorDesc& A = out[2];
    if (A.dtype != DType::kI32 || A.rank() != 1 || !A.contiguous || A.shape[0] != Z.shape[0]) return false;
  }
  return true;
}
template <DType kDt>
bool softmax_ce_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return softmax_ce_check<kDt>(in, ni, out, no);
}
template <typename T, int kPackets>
Status launch_ce_cluster(int nranks, int slice, const T* z, const int32_t* lab, T* dz, float* loss, int32_t* am, int64_t B,
                         int64_t C, float scale, cudaStream_t stream) {
  const int64_t max_clusters = static_cast<int64_t>(sm_count()) * kStreamBlocksPerSm / nranks;
  const int64_t clusters = B < max_clusters ? B : max_clusters;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(nranks);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * nranks));
  cfg.blockDim = dim3(kClusterThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaGetLastError();
  if (cudaLaunchKernelEx(&cfg, softmax_ce_cluster_kernel<T, kPackets>, z, lab, dz, loss, am, B, C, scale, slice) != cudaSuccess) {
    cudaGetLastError();
    return Status::Internal;
  }
  return launch_status();
}

template <DType kDt, typename T>
Status softmax_ce_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                         cudaStream_t stream) {
  if (!softmax_ce_check<kDt>(in, ni, out, no)) return Status::InvalidArgument;
  const int64_t B = in[0].shape[0], C = in[0].shape[1];
  float scale = 1.0f / static_cast<float>(B);
  read_attr_payload(attr, schema::kSoftmaxCE, false, &scale, 4);
  const T* z = static_cast<const T*>(in[0].data);
  const int32_t* lab = static_cast<const int32_t*>(in[1].data);
  T* dz = static_cast<T*>(out[0].data);
  float* loss = static_cast<float*>(out[1].data);
  int32_t* am = no == 3 ? static_cast<int32_t*>(out[2].data) : nullptr;
  constexpr int kN = Pack16<T>::kN;
  constexpr int kMaxPk = sizeof(T) == 4 ? 8 : 4;
  const bool vec = (C % kN == 0) && aligned_to(z, 16) && aligned_to(dz, 16);
  const size_t smem = row_pipe_smem(C * static_cast<int64_t>(sizeof(T)));
  const RowCfg c = (vec && smem <= kMaxRowPipeSmem) ? pick_row_cfg(C / kN, kMaxPk) : RowCfg{};
  cudaGetLastError();
  // Rows too long for one block's registers (more than 32768 fp32 columns) go one row per cluster of up to 8 small CTAs
  // and stay single-pass up to 65536 columns ([4096,65536] f32: 3712 GB/s against 1383 for the three-read fallback).
  // Where one block can hold the row, the persistent pipelined kernel is faster ([8192,32000] f32: 6318 GB/s against
  // 4010 as clusters of four: a cluster lives for one row, and its launch, its load latency and its three cluster
  // barriers are exposed at four resident CTAs per SM). AICF_CE_CLUSTER=0|1 (tuning, read once per process) forces the
  // choice wherever the row can be split that way.
  static const int cluster_override = [] {
    const char* e = std::getenv("AICF_CE_CLUSTER");
    return (e == nullptr || e[0] == 0) ? -1 : (e[0] == '0' ? 0 : 1);
  }();
  const int64_t row_packets = C / kN;
  if (vec && (cluster_override >= 0 ? cluster_override != 0 : c.packets == 0)) {
    // AICF_CE_CLUSTER_PACKETS=n (tuning, read once per process): packets a thread may hold before the cluster grows
    static const int pk_limit = [] {
      const char* e = std::getenv("AICF_CE_CLUSTER_PACKETS");
      const int v = e ? std::atoi(e) : 0;
      return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 0;
    }();
    // 64 registers hold 32 fp32 elements per thread, or 16 elements of a 16-bit type next to their packed form
    constexpr int kClusterMaxPk = sizeof(T) == 4 ? 8 : 2;
    const int64_t per_cta_max =
        static_cast<int64_t>(kClusterThreads) * (pk_limit > 0 && pk_limit < kClusterMaxPk ? pk_limit : kClusterMaxPk);
    int nranks = 2;
    while (nranks < 8 && (row_packets + nranks - 1) / nranks > per_cta_max) nranks *= 2;
    const int64_t slice = (row_packets + nranks - 1) / nranks;
    if (slice <= per_cta_max && row_packets >= nranks) {
      const int64_t per = (slice + kClusterThreads - 1) / kClusterThreads;
      const int sl = static_cast<int>(slice);
      if (per <= 1) return launch_ce_cluster<T, 1>(nranks, sl, z, lab, dz, loss, am, B, C, scale, stream);
      if (per <= 2) return launch_ce_cluster<T, 2>(nranks, sl, z, lab, dz, loss, am, B, C, scale, stream);
      if constexpr (sizeof(T) == 4) {
        if (per <= 4) return launch_ce_cluster<T, 4>(nranks, sl, z, lab, dz, loss, am, B, C, scale, stream);
        return launch_ce_cluster<T, 8>(nranks, sl, z, lab, dz, loss, am, B, C, scale, stream);
      }
    }
  }
  if (c.packets == 0) {
    softmax_ce_multipass_kernel<T><<<streaming_grid(B, 1, 8), 256, 0, stream>>>(z, lab, dz, loss, am, B, C, scale);
    return launch_status();
  }
  bool ok_attr = true;
  // The two-barrier form is the default everywhere. AICF_CE_LOCKSTEP=1 selects the lockstep form (tuning; read once
  // per process): it used to win for one 1024-thread block per SM, and lost that once the per-element arg-max and
  // one-hot work left the loops ([8192,32000] f32: 6396 GB/s against 5612 in lockstep).
  static const bool lockstep = [] {
    const char* e = std::getenv("AICF_CE_LOCKSTEP");
    return e != nullptr && e[0] == '1';
  }();
  const bool full = use_full_rows(C / kN == static_cast<int64_t>(c.threads) * c.packets, sizeof(T));
  const size_t smem_launch = row_smem_capped_residency(smem, c.threads);  // the grid is still sized from `smem`
  // AICF_CE_EARLY_REFILL=0|1 (tuning, read once per process); default: when an SM holds one block. GB/s without / with:
  // [8192,32000] f32 (one block per SM) 6322 / 6550; [16384,16384] (two) 5760 / 5560; [16384,8192] 6243 / 6317;
  // [65536,1024] 6375 / 5975.
  static const int early_override = [] {
    const char* e = std::getenv("AICF_CE_EARLY_REFILL");
    return (e == nullptr || e[0] == 0) ? -1 : (e[0] == '0' ? 0 : 1);
  }();
  const int early_refill = early_override >= 0 ? early_override : (row_pipe_blocks_per_sm(c.threads, smem_launch) == 1 ? 1 : 0);
#define AICF_CE_LAUNCH_M(PK, LS, FULL, EARLY)                                                                              \
  if ((ok_attr = allow_smem(softmax_ce_regs_kernel<T, PK, LS, FULL, EARLY>, smem_launch)))                                 \
    softmax_ce_regs_kernel<T, PK, LS, FULL, EARLY>                                                                         \
        <<<streaming_grid(B, 1, row_blocks_per_sm(softmax_ce_regs_kernel<T, PK, LS, FULL, EARLY>, c.threads, smem)),       \
           c.threads, smem_launch, stream>>>(z, lab, dz, loss, am, B, C, scale)
#define AICF_CE_LAUNCH(PK)                                                \
  if (lockstep) { AICF_CE_LAUNCH_M(PK, true, false, false); }             \
  else if (early_refill) {                                                \
    if (full) { AICF_CE_LAUNCH_M(PK, false, true, true); }                \
    else { AICF_CE_LAUNCH_M(PK, false, false, true); }                    \
  } else if (full) { AICF_CE_LAUNCH_M(PK, false, true, false); }          \
  else { AICF_CE_LAUNCH_M(PK, false, false, false); }
  switch (c.packets) {
    case 1: AICF_CE_LAUNCH(1); break;
    case 2: AICF_CE_LAUNCH(2); break;
    case 4: AICF_CE_LAUNCH(4); break;
    default: AICF_CE_LAUNCH(kMaxPk); break;
  }
#undef AICF_CE_LAUNCH
#undef AICF_CE_LAUNCH_M
  if (!ok_attr) {
    cudaGetLastError();
    return Status::Internal;
  }
  return launch_status();
}

size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }
using LaunchFn = Status (*)(const TensorDesc*, int, TensorDesc*, int, const void*, void*, size_t, cudaStream_t);
using SupportedFn = bool (*)(const TensorDesc*, int, const TensorDesc*, int, const void*);
KernelVariant make(const char* name, LaunchFn l, SupportedFn s) {
  KernelVariant v{};
  v.name = name;
  v.flags = kKV_CaptureSafe;
  v.launch = l;
  v.supported = s;
  v.query_workspace = no_workspace;
  return v;
}

}  // namespace

// Reads (optionally clears) the status word of the row pipeline's bounded waits. Synchronises the device.
int row_pipeline_status(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_row_pipeline_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (clear && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_row_pipeline_status, &zero, sizeof(int));
  }
  return v;
}

KernelVariant make_softmax_lastdim_f32_variant() { return make("softmax_f32_sm100", softmax_launch<DType::kF32, float>, softmax_supported<DType::kF32>); }
KernelVariant make_softmax_lastdim_bf16_variant() { return make("softmax_bf16_sm100", softmax_launch<DType::kBF16, __nv_bfloat16>, softmax_supported<DType::kBF16>); }
KernelVariant make_softmax_lastdim_f16_variant() { return make("softmax_f16_sm100", softmax_launch<DType::kF16, __half>, softmax_supported<DType::kF16>); }
KernelVariant make_softmax_ce_f32_variant() { return make("softmax_ce_f32_sm100", softmax_ce_launch<DType::kF32, float>, softmax_ce_supported<DType::kF32>); }
KernelVariant make_softmax_ce_bf16_variant() { return make("softmax_ce_bf16_sm100", softmax_ce_launch<DType::kBF16, __nv_bfloat16>, softmax_ce_supported<DType::kBF16>); }
KernelVariant make_softmax_ce_f16_variant() { return make("softmax_ce_f16_sm100", softmax_ce_launch<DType::kF16, __half>, softmax_ce_supported<DType::kF16>); }

}  // namespace aicf::cuda
