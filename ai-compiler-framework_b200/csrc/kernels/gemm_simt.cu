// Tiled SIMT GEMM with fused bias/ReLU epilogue: fp32 FFMA accumulate, arbitrary operand strides,
// operands in f32 / f16 / bf16, output in f32 / f16 / bf16.
//
// Role: (1) the exact-fp32 contraction (the tensor cores have no IEEE fp32 mode; the reference's fp32
// kernel ops/gemm/launcher.cu:155-172 accumulates with one FMA per k in increasing k, and so does this
// kernel, per output element, so results agree bit for bit); (2) shapes the TMA path cannot take
// (rows not 16-byte aligned, tiny problems).
//
// 256 threads, register-staged double buffering, four tile shapes with BM*BK = BN*BK = 1024 (every thread stages
// four elements of each operand per k-step): 128x128x8 with 8x8 outputs per thread for large problems, then
// 64x64x16 (4x4), 32x32x32 (2x2) and 16x16x64 (1x1). The launcher takes the largest tile that still yields at
// least one block per SM: a 64x256x784 product is 2 blocks of the large tile (142 us, two SMs busy) but 64 blocks
// of the smallest (a few us). The order of the k loop per output element is the same in all of them.
#include <type_traits>

#include "gemm_common.cuh"

namespace aicf::cuda {

namespace {


__device__ __forceinline__ float load_elem(const void* base, int64_t idx, DType dt) {
  switch (dt) {
    case DType::kF32: return static_cast<const float*>(base)[idx];
    case DType::kF16: return __half2float(static_cast<const __half*>(base)[idx]);
    case DType::kBF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    default: return 0.0f;
  }
}
__device__ __forceinline__ void store_elem(void* base, int64_t idx, DType dt, float v) {
  switch (dt) {
    case DType::kF32: static_cast<float*>(base)[idx] = v; break;
    case DType::kF16: static_cast<__half*>(base)[idx] = __float2half_rn(v); break;
    case DType::kBF16: static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v); break;
    default: break;
  }
}

struct SimtArgs {
  const void *A, *B, *bias, *mask;
  void* C;
  int64_t mask_ld;
  int64_t Ars, Acs, Brs, Bcs, Crs, Ccs, bias_stride;
  int M, N, K;
  DType dtA, dtB, dtC, dtBias;
  int relu;
  int a_k_fast, b_n_fast;  // which index consecutive threads walk when loading (coalescing)
};

template <typename TIn>
__device__ __forceinline__ float ld_in(const void* base, int64_t idx) {
  return Cvt<TIn>::to_f(static_cast<const TIn*>(base)[idx]);
}

template <typename TIn, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtArgs g) {
  static_assert(BM * BK == 1024 && BN * BK == 1024 && (BM / TM) * (BN / TN) == 256, "256 threads, 4 staged elements each");
  // Row padding keeps the k-fast staging writes off a single bank; it is a multiple of the vector width of the reads.
  constexpr int PADA = TM >= 4 ? 4 : TM, PADB = TN >= 4 ? 4 : TN;
  __shared__ __align__(16) float As[2][BK][BM + PADA];
  __shared__ __align__(16) float Bs[2][BK][BN + PADB];
  const int tid = threadIdx.x;
  constexpr int kTX = BN / TN;
  const int tx = tid % kTX, ty = tid / kTX;  // thread owns rows ty*TM.., cols tx*TN..
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  // each thread stages 4 elements of the A tile (BM x BK) and 4 of the B tile (BK x BN)
  int am[4], ak[4], bk[4], bn[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = tid + i * 256;
    if (g.a_k_fast) { ak[i] = e % BK; am[i] = e / BK; } else { am[i] = e % BM; ak[i] = e / BM; }
    if (g.b_n_fast) { bn[i] = e % BN; bk[i] = e / BN; } else { bk[i] = e % BK; bn[i] = e / BK; }
  }
  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + am[i], k = k0 + ak[i];
      ra[i] = (m < g.M && k < g.K) ? ld_in<TIn>(g.A, m * g.Ars + k * g.Acs) : 0.0f;
      const int kk = k0 + bk[i], n = n0 + bn[i];
      rb[i] = (kk < g.K && n < g.N) ? ld_in<TIn>(g.B, kk * g.Brs + n * g.Bcs) : 0.0f;
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[buf][ak[i]][am[i]] = ra[i];
      Bs[buf][bk[i]][bn[i]] = rb[i];
    }
  };
  auto load_vec = [](float* dst, const float* src, auto n_tag) {
    constexpr int n = decltype(n_tag)::value;
    if constexpr (n == 8) {
      *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
      *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
    } else if constexpr (n == 4) {
      *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
    } else if constexpr (n == 2) {
      *reinterpret_cast<float2*>(dst) = *reinterpret_cast<const float2*>(src);
    } else {
      dst[0] = src[0];
    }
  };

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < g.K; k0 += BK) {
    const bool more = k0 + BK < g.K;
    if (more) fetch(k0 + BK);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
      load_vec(a, &As[buf][k][ty * TM], std::integral_constant<int, TM>{});
      load_vec(b, &Bs[buf][k][tx * TN], std::integral_constant<int, TN>{});
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (more) {
      stage(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.bias) v += load_elem(g.bias, n * g.bias_stride, g.dtBias);
      if (g.relu) v = v > 0.0f ? v : 0.0f;
      if (g.mask && !(load_elem(g.mask, m * g.mask_ld + n, g.dtC) > 0.0f)) v = 0.0f;
      store_elem(g.C, m * g.Crs + n * g.Ccs, g.dtC, v);
    }
  }
}

}  // namespace

Status gemm_simt_run(const GemmProblem& p, cudaStream_t stream) {
  if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.K > 0x7fffffff) return Status::NotImplemented;
  if (p.A.dtype != p.B.dtype) return Status::InvalidArgument;
  SimtArgs g{};
  g.A = p.A.data; g.B = p.B.data; g.C = const_cast<void*>(p.C.data); g.bias = p.bias;
  g.Ars = p.A.rs; g.Acs = p.A.cs; g.Brs = p.B.rs; g.Bcs = p.B.cs; g.Crs = p.C.rs; g.Ccs = p.C.cs;
  g.bias_stride = p.bias_stride;
  g.mask = p.mask;
  g.mask_ld = p.mask_ld;
  g.M = static_cast<int>(p.M); g.N = static_cast<int>(p.N); g.K = static_cast<int>(p.K);
  g.dtA = p.A.dtype; g.dtB = p.B.dtype; g.dtC = p.C.dtype; g.dtBias = p.bias_dtype;
  g.relu = p.relu ? 1 : 0;
  g.a_k_fast = p.A.cs <= p.A.rs;
  g.b_n_fast = p.B.cs <= p.B.rs;
  // Largest tile that gives every SM a block; the smallest tile when even that one does not.
  const int64_t sms = sm_count();
  auto blocks = [&](int64_t bm, int64_t bn) { return ((p.M + bm - 1) / bm) * ((p.N + bn - 1) / bn); };
  const int tile = blocks(128, 128) >= sms ? 128 : blocks(64, 64) >= sms ? 64 : blocks(32, 32) >= sms ? 32 : 16;
  cudaGetLastError();
#define AICF_SIMT_LAUNCH(TIN)                                                                                   \
  switch (tile) {                                                                                               \
    case 128: gemm_simt_kernel<TIN, 128, 128, 8, 8, 8><<<grid_for(128, 128), 256, 0, stream>>>(g); break;         \
    case 64: gemm_simt_kernel<TIN, 64, 64, 16, 4, 4><<<grid_for(64, 64), 256, 0, stream>>>(g); break;             \
    case 32: gemm_simt_kernel<TIN, 32, 32, 32, 2, 2><<<grid_for(32, 32), 256, 0, stream>>>(g); break;             \
    default: gemm_simt_kernel<TIN, 16, 16, 64, 1, 1><<<grid_for(16, 16), 256, 0, stream>>>(g); break;             \
  }
  auto grid_for = [&](int64_t bm, int64_t bn) {
    return dim3(static_cast<unsigned>((p.N + bn - 1) / bn), static_cast<unsigned>((p.M + bm - 1) / bm));
  };
  switch (p.A.dtype) {
    case DType::kF32: AICF_SIMT_LAUNCH(float); break;
    case DType::kF16: AICF_SIMT_LAUNCH(__half); break;
    case DType::kBF16: AICF_SIMT_LAUNCH(__nv_bfloat16); break;
    default: return Status::InvalidArgument;
  }
#undef AICF_SIMT_LAUNCH
  return launch_status();
}

}  // namespace aicf::cuda
