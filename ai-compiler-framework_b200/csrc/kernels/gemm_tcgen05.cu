// Dense GEMM for Blackwell (sm_100a): C = [relu](op(A) * op(B) [+ bias]) with 16-bit operands
// (bf16 or f16), fp32 accumulation in tensor memory, output bf16 / f16 / f32; and, under opt-in kernel ids, fp32
// operands as three TF32 products per k step (section "3xTF32" below).
//
// Three kernels share the helpers of this file:
//   gemm_tcgen05_2cta_kernel   CTA pairs (clusters of 2) on 256x256 tiles with tcgen05.mma.cta_group::2; the default
//                              for problems with enough tiles to occupy the SM pairs
//   gemm_tcgen05_kernel<TN>    one CTA per 128 x TN tile, TN = 256 / 128 / 64 (4 / 6 / 8 stages): small problems
//   gemm_tf32x3_kernel         one CTA per 128x128 tile, kind::tf32, hi/lo operand parts staged by tf32_split_kernel
//
// Structure of each (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D tile loads (no multicast) into a ring of 128B-swizzled
//               shared-memory tiles, completion on mbarriers
//   warp 1      owns tensor memory (tcgen05.alloc / dealloc) and issues tcgen05.mma from one elected lane;
//               tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator (each warp its own 32-lane TMEM sub-partition),
//               + bias, ReLU (or the ReLU-backward mask), convert, 16-byte global stores
// Two (3xTF32: four) accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of tile i+1. All
// four transpose combinations are handled without moving data: an operand whose contiguous dimension is M/N instead
// of K is loaded as 64x64 boxes and described to the MMA as "MN-major" through the shared-memory and instruction
// descriptors (the 3xTF32 path gets K-major operands from its split pre-pass instead).
//
// Every wait is bounded: after ~1 s without progress a role raises the CTA's abort flag, records a
// code in the device status word, everybody leaves their loops, tensor memory is released and the
// kernel returns normally. The host reads the word through gemm_tcgen05_status().
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "gemm_common.cuh"

namespace aicf::cuda {

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 64;   // 64 x 2 bytes = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kAStageBytes = kTileM * kTileK * 2;   // 16 KiB
constexpr int kBStageBytes = kTileN * kTileK * 2;   // 32 KiB
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kChunkBytes = 64 * kTileK * 2;        // one 64x64 box = 8 KiB (MN-major operands)
constexpr int kAccBufs = 2;
constexpr int kTmemCols = 512;
constexpr int kThreads = 192;
constexpr int kGroupM = 16;   // tile rasterisation: 16 row-tiles share their column tiles in L2
constexpr int kDefaultCStream = 0;  // C stores: 0 = default write-back, 1 = streaming (evict-first)
constexpr int kDefaultAbHint = 0;   // operand loads of the paired kernel: no L2 eviction hint
constexpr unsigned long long kWaitBudgetNs = 1000000000ull;


__device__ int g_gemm_status = 0;  // 0 ok; otherwise (role << 8) | reason of the first CTA that gave up

// Optional timeline of CTA 0 (nanoseconds from %globaltimer), for tuning. Off unless the host enables it.
//  [0] kernel start  [1] set-up done  [2] first TMA issued  [3] first stage landed  [4] first tile's MMAs issued
//  [5] first accumulator ready  [6] first tile stored  [7] last tile stored  [8] kernel end
//  [9] MMA wait-for-data ns  [10] MMA wait-for-accumulator ns  [11] producer wait-for-slot ns
//  [12] epilogue wait-for-accumulator ns  [13] epilogue busy ns  [14] tiles done by CTA 0
__device__ int g_gemm_timeline_on = 0;
__device__ unsigned long long g_gemm_timeline[16];

struct GemmParams {
  void* C;
  const void* bias;
  const void* mask;     // optional ReLU-backward mask, dtype of C, row pitch mask_ld elements
  int64_t mask_ld;
  int mask_vec_ok;      // mask rows allow 16-byte loads
  int64_t ldc;          // elements
  int64_t bias_stride;  // elements
  int M, N, K;
  int c_dtype;          // DType value of C
  int bias_dtype;       // DType value of bias (0 = none)
  int relu;
  int a_mn_major, b_mn_major;
  uint32_t idesc;
  int c_vec_ok;         // C rows allow 16-byte stores
  // split-K (single-CTA kernel only): `splits` CTAs share a tile, each accumulating a contiguous range of k blocks
  // and writing its raw fp32 accumulator to partial[split][M][N]; splitk_finish_kernel adds the parts in split order
  // and applies the epilogue. splits <= 1: the kernel stores C itself.
  int splits;
  float* partial;
  // tuning (launcher defaults, AICF_GEMM_* overrides): rasterisation group in 128-row tiles, streaming (evict-first)
  // stores of C, and L2 eviction hints on the operand loads (bit 0 / 1: A / B evict_last, bit 2 / 3: A / B evict_first)
  int group_m;
  int c_stream;
  int ab_hint;
  // paired kernel: last, partly filled round of tiles done as 256x128 half tiles (see PairItem)
  int tail_halves;
  uint32_t idesc_half;  // instruction descriptor with N = 128
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait. Returns false when the CTA is aborting (flag raised here on timeout or elsewhere).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int who) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0u) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, (who << 8) | 1);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"  // same asm statement: the registers are not readable before the wait
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
//   K-major : rows of 128 B (64 elements of K); SBO = 1024 B between 8-row groups; LBO unused (1)
//   MN-major: 64-element MN chunks of 64 k-rows x 128 B; LBO = 8192 B between chunks,
//             SBO = 1024 B between 8-k groups
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, int mn_major) {
  const uint64_t lbo = mn_major ? (kChunkBytes >> 4) : 1;
  const uint64_t sbo = 1024 >> 4;
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int* tm, int* tn, int group_m = kGroupM) {
  const int per_group = group_m * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int in_group = tile - group * per_group;
  *tm = first_m + in_group % rows;
  *tn = in_group / rows;
}

__device__ __forceinline__ float bias_at(const GemmParams& p, int col) {
  if (p.bias_dtype == static_cast<int>(DType::kF32)) return __ldg(static_cast<const float*>(p.bias) + col * p.bias_stride);
  if (p.bias_dtype == static_cast<int>(DType::kBF16))
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col * p.bias_stride]);
  return __half2float(static_cast<const __half*>(p.bias)[col * p.bias_stride]);
}

// Two adjacent 32-column chunks in one go: both loads are in flight together, one wait.
__device__ __forceinline__ void tmem_ld_32x32_pair(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}

// One thread's 32 consecutive output columns of one row: + bias (from shared memory), ReLU, convert, store.
// Every array index is a compile-time constant so the values stay in registers.
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, int row, int col0, const uint32_t* r,
                                               const float* bias_s) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) + bias_s[j];
  if (p.relu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
  }
  if (row >= p.M) return;
  const int64_t off = static_cast<int64_t>(row) * p.ldc + col0;
  const bool full_chunk = (col0 + 32 <= p.N) && p.c_vec_ok;
  if (p.mask) {  // dX = (Y > 0) ? acc : 0, Y read in C's dtype
    const int64_t moff = static_cast<int64_t>(row) * p.mask_ld + col0;
    const bool full_mask = (col0 + 32 <= p.N) && p.mask_vec_ok;
    if (p.c_dtype == static_cast<int>(DType::kF32)) {
      const float* ms = static_cast<const float*>(p.mask) + moff;
      if (full_mask) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 y = __ldcs(reinterpret_cast<const float4*>(ms) + q);
          if (!(y.x > 0.0f)) v[4 * q] = 0.0f;
          if (!(y.y > 0.0f)) v[4 * q + 1] = 0.0f;
          if (!(y.z > 0.0f)) v[4 * q + 2] = 0.0f;
          if (!(y.w > 0.0f)) v[4 * q + 3] = 0.0f;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N && !(ms[j] > 0.0f)) v[j] = 0.0f;
      }
    } else {
      // "y > 0" on the raw 16-bit pattern: sign clear, magnitude non-zero and not above infinity (NaN fails, as it
      // does in the float comparison). bf16 and f16 differ only in the bit pattern of infinity.
      const uint32_t inf_bits = p.c_dtype == static_cast<int>(DType::kBF16) ? 0x7F80u : 0x7C00u;
      auto not_positive = [inf_bits](uint32_t y) {
        const uint32_t mag = y & 0x7FFFu;
        return (y & 0x8000u) != 0u || mag == 0u || mag > inf_bits;
      };
      const uint16_t* ms = static_cast<const uint16_t*>(p.mask) + moff;
      if (full_mask) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 y = __ldcs(reinterpret_cast<const uint4*>(ms) + q);
          const uint32_t w[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t lo = w[e] & 0xFFFFu, hi = w[e] >> 16;
            if (not_positive(lo)) v[8 * q + 2 * e] = 0.0f;
            if (not_positive(hi)) v[8 * q + 2 * e + 1] = 0.0f;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) {
            if (not_positive(ms[j])) v[j] = 0.0f;
          }
      }
    }
  }
  if (p.c_dtype == static_cast<int>(DType::kF32)) {
    float* dst = static_cast<float*>(p.C) + off;
    if (full_chunk) {
      if (p.c_stream) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          __stcs(reinterpret_cast<float4*>(dst) + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          reinterpret_cast<float4*>(dst)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = v[j];
    }
    return;
  }
  uint32_t packed[16];
  if (p.c_dtype == static_cast<int>(DType::kBF16)) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      packed[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      packed[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  uint16_t* dst = static_cast<uint16_t*>(p.C) + off;
  if (full_chunk) {
    if (p.c_stream) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        __stcs(reinterpret_cast<uint4*>(dst) + q, make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]));
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        reinterpret_cast<uint4*>(dst)[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) dst[j] = static_cast<uint16_t>((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xFFFFu));
  }
}

// ------------------------------------------------------------------ kernel
// TN = tile width (256, 128 or 64 columns). Narrow tiles are for problems with too few 128x256 tiles to occupy the
// SMs: more CTAs, a shorter epilogue per CTA and a deeper ring in the same shared memory.
template <int TN> struct SingleCfg {
  static constexpr int kSt = TN == 256 ? 4 : TN == 128 ? 6 : 8;     // ring depth
  static constexpr int kStB = kAStageBytes + TN * kTileK * 2;        // bytes per stage
  static constexpr int kTm = 2 * TN;                                 // TMEM columns: two accumulators
  static constexpr size_t kSmem = 1024 + size_t(kSt) * kStB + 256 + 4 * TN * sizeof(float);
};

template <int TN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const GemmParams p) {
  constexpr int kSt = SingleCfg<TN>::kSt, kStB = SingleCfg<TN>::kStB, kTm = SingleCfg<TN>::kTm;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128B swizzle atoms repeat every 1024 B
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bars = base + kSt * kStB;
  // barrier map (8 B each): full[kSt], empty[kSt], acc_full[0..1], acc_empty[0..1]
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kSt, bar_acc_full = bars + 16 * kSt,
                 bar_acc_empty = bars + 16 * kSt + 8 * kAccBufs;
  uint8_t* misc = base_ptr + kSt * kStB + 16 * kSt + 16 * kAccBufs;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
  float* bias_smem = reinterpret_cast<float*>(base_ptr + kSt * kStB + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kTileM - 1) / kTileM, tiles_n = (p.N + TN - 1) / TN;
  const int splits = p.splits > 1 ? p.splits : 1;
  const int num_tiles = tiles_m * tiles_n * splits;  // work items: (tile, split), split fastest
  const int k_blocks_all = (p.K + kTileK - 1) / kTileK;
  const int kb_per_split = (k_blocks_all + splits - 1) / splits;

  const bool tl = g_gemm_timeline_on != 0 && blockIdx.x == 0;
  if (tl && threadIdx.x == 0) g_gemm_timeline[0] = global_ns();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSt; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTm);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  if (tl && threadIdx.x == 0) g_gemm_timeline[1] = global_ns();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      unsigned long long waited = 0;
      bool first = true;
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile / splits, tiles_m, tiles_n, &tm, &tn, p.group_m);
        const int m0 = tm * kTileM, n0 = tn * TN;
        const int kb_lo = (tile % splits) * kb_per_split, kb_hi = min(kb_lo + kb_per_split, k_blocks_all);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          const unsigned long long w0 = tl ? global_ns() : 0;
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1)) { alive = false; break; }
          if (tl) {
            waited += global_ns() - w0;
            if (first) { g_gemm_timeline[2] = global_ns(); first = false; }
          }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = base + stage * kStB, sb = sa + kAStageBytes;
          const int k0 = kb * kTileK;
          mbar_expect_tx(full, kStB);
          if (p.a_mn_major) {
            tma_load_2d(sa, &tmap_a, m0, k0, full);
            tma_load_2d(sa + kChunkBytes, &tmap_a, m0 + 64, k0, full);
          } else {
            tma_load_2d(sa, &tmap_a, k0, m0, full);
          }
          if (p.b_mn_major) {
#pragma unroll
            for (int j = 0; j < TN / 64; ++j) tma_load_2d(sb + j * kChunkBytes, &tmap_b, n0 + 64 * j, k0, full);
          } else {
            tma_load_2d(sb, &tmap_b, k0, n0, full);
          }
          if (++stage == kSt) { stage = 0; phase ^= 1u; }
        }
      }
      if (tl) g_gemm_timeline[11] = waited;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      const uint32_t a_step = p.a_mn_major ? (2 * 1024) >> 4 : (kUmmaK * 2) >> 4;  // descriptor units of 16 B
      const uint32_t b_step = p.b_mn_major ? (2 * 1024) >> 4 : (kUmmaK * 2) >> 4;
      unsigned long long wait_data = 0, wait_acc = 0;
      bool first = true, first_tile = true;
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        unsigned long long w0 = tl ? global_ns() : 0;
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, 2)) { alive = false; break; }
        if (tl) wait_acc += global_ns() - w0;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * TN;
        const int kb_lo = (tile % splits) * kb_per_split, kb_hi = min(kb_lo + kb_per_split, k_blocks_all);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          w0 = tl ? global_ns() : 0;
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3)) { alive = false; break; }
          if (tl) {
            wait_data += global_ns() - w0;
            if (first) { g_gemm_timeline[3] = global_ns(); first = false; }
          }
          tc_fence_after();
          const uint32_t sa = base + stage * kStB, sb = sa + kAStageBytes;
          const uint64_t adesc = make_smem_desc(sa, p.a_mn_major);
          const uint64_t bdesc = make_smem_desc(sb, p.b_mn_major);
#pragma unroll
          for (int k = 0; k < kTileK / kUmmaK; ++k)
            umma_f16(tmem_d, adesc + k * a_step, bdesc + k * b_step, p.idesc, (kb != kb_lo || k != 0) ? 1u : 0u);
          umma_commit(bar_empty + 8 * stage);  // stage is free once these MMAs have read it
          if (++stage == kSt) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit(bar_acc_full + 8 * acc);   // accumulator complete
        if (tl && first_tile) { g_gemm_timeline[4] = global_ns(); first_tile = false; }
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
      if (tl) { g_gemm_timeline[9] = wait_data; g_gemm_timeline[10] = wait_acc; }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int sub = warp & 3;  // TMEM sub-partition this warp may read: lanes [32*sub, 32*sub+32)
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    const bool tle = tl && warp == 2 && lane == 0;
    unsigned long long e_wait = 0, e_busy = 0, e_tiles = 0;
    // With split-K the epilogue only parks the raw accumulator: fp32, no bias, no activation, packed [M][N] rows.
    GemmParams q = p;
    if (splits > 1) {
      q.ldc = p.N;
      q.c_dtype = static_cast<int>(DType::kF32);
      q.bias_dtype = 0;
      q.relu = 0;
      q.mask = nullptr;
      q.c_vec_ok = (p.N % 4) == 0;
    }
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile / splits, tiles_m, tiles_n, &tm, &tn, p.group_m);
      const int row = tm * kTileM + sub * 32 + lane;
      const int n0 = tn * TN;
      if (splits > 1) q.C = p.partial + static_cast<int64_t>(tile % splits) * p.M * p.N;
      const unsigned long long e0 = tle ? global_ns() : 0;
      // the TMEM loads below are warp-collective: the whole warp proceeds or the whole warp leaves
      if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, 4))) { alive = false; break; }
      tc_fence_after();
      const unsigned long long e1 = tle ? global_ns() : 0;
      if (tle) {
        e_wait += e1 - e0;
        if (e_tiles == 0) g_gemm_timeline[5] = e1;
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(sub * 32) << 16) + acc * TN;
      // bias of this tile's 256 columns -> this warp's private strip of shared memory (no cross-warp barrier,
      // so a warp that gives up on a wait can never leave another one stuck)
      float* bs = bias_smem + (warp - 2) * TN;
#pragma unroll
      for (int h = 0; h < TN / 32; ++h) {
        const int col = n0 + lane + 32 * h;
        bs[lane + 32 * h] = (q.bias_dtype != 0 && col < p.N) ? bias_at(p, col) : 0.0f;
      }
      __syncwarp();
#pragma unroll 1
      for (int c = 0; c < TN / 32; c += 2) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[64];
        const bool two = col0 + 32 < p.N;  // warp-uniform
        if (two) {
          tmem_ld_32x32_pair(taddr + c * 32, r);
        } else {
          tmem_ld_32x32(taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        }
        epilogue_chunk(q, row, col0, &r[0], bs + c * 32);
        if (two) epilogue_chunk(q, row, col0 + 32, &r[32], bs + c * 32 + 32);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      if (tle) {
        const unsigned long long e2 = global_ns();
        e_busy += e2 - e1;
        if (e_tiles == 0) g_gemm_timeline[6] = e2;
        g_gemm_timeline[7] = e2;
        ++e_tiles;
      }
    }
    if (tle) { g_gemm_timeline[12] = e_wait; g_gemm_timeline[13] = e_busy; g_gemm_timeline[14] = e_tiles; }
  }

  // ---------------- teardown ----------------
  if (*abort_flag) {
    // error path only: give loads that may still be in flight time to land before smem is released
    for (int i = 0; i < 64; ++i) __nanosleep(16384);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTm);
  }
  if (tl && threadIdx.x == 0) g_gemm_timeline[8] = global_ns();
}

// ================================================================== paired-CTA variant (cta_group::2)
// Two CTAs of a cluster work on one 256x256 tile: CTA r holds rows [128r, 128r+128) of A and columns
// [128r, 128r+128) of B in its shared memory, one tcgen05.mma.cta_group::2 issued by the leader (rank 0) reads
// both CTAs' operands and writes 128 accumulator lanes x 256 columns in each CTA's tensor memory. Per CTA a
// k-step moves 32 KiB instead of 48 KiB, so the same shared memory holds a 6-stage ring: less L2->SM traffic
// and more latency cover. Loads carry no multicast: each CTA issues its own cp.async.bulk.tensor (cta_group::2
// form, whose completion may signal the leader's mbarrier).
constexpr int k2Stages = 6;
constexpr int k2HalfN = kTileN / 2;                       // B columns held per CTA
constexpr int k2AStageBytes = kTileM * kTileK * 2;        // 16 KiB
constexpr int k2BStageBytes = k2HalfN * kTileK * 2;       // 16 KiB
constexpr int k2StageBytes = k2AStageBytes + k2BStageBytes;
constexpr size_t k2SmemBytes = 1024 + size_t(k2Stages) * k2StageBytes + 256 + 4 * kTileN * sizeof(float);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address of this CTA's window) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar_cluster)
      : "memory");
}
// Same load with an L2 eviction policy (from createpolicy) attached.
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar_cluster), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 0x3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(both)
               : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m2, int tiles_n, int* tm, int* tn, int group_m) {
  const int kGroup = max(group_m / 2, 1);  // default 8 pair-rows = 16 row tiles of 128
  const int per_group = kGroup * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * kGroup;
  const int rows = min(kGroup, tiles_m2 - first_m);
  const int in_group = tile - group * per_group;
  *tm = first_m + in_group % rows;
  *tn = in_group / rows;
}

// Work items of the paired kernel. Clusters take items round-robin, so `num_tiles` tiles on `num_clusters` clusters
// run in ceil(num_tiles / num_clusters) rounds and the last round may be mostly empty (4096^3: 256 tiles on 74
// clusters = 3 full rounds + 34 tiles). When the left-over tiles number at most half the clusters, each of them is
// split into its two 256x128 column halves: twice as many items, each about half as long, still one round - the
// tail costs half a round instead of a whole one. Items [0, full) are whole tiles, the rest are halves.
struct PairItem {
  int tile;    // 256x256 tile index (rasterised by pair_tile_coords)
  int half;    // 0 / 1: column half, when `width` is 128
  int width;   // 256 or 128 columns
};
struct PairSchedule {
  int full, items;
  __device__ __forceinline__ PairSchedule(int num_tiles, int num_clusters, int tail_halves) {
    const int rem = num_tiles % num_clusters;
    const bool halve = tail_halves != 0 && rem > 0 && 2 * rem <= num_clusters;
    full = halve ? num_tiles - rem : num_tiles;
    items = full + (halve ? 2 * rem : 0);
  }
  __device__ __forceinline__ PairItem at(int w) const {
    if (w < full) return PairItem{w, 0, kTileN};
    const int h = w - full;
    return PairItem{full + (h >> 1), h & 1, kTileN / 2};
  }
};

__global__ void __launch_bounds__(kThreads, 1)
    gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             const __grid_constant__ CUtensorMap tmap_b_half, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bars = base + k2Stages * k2StageBytes;
  // barrier map (8 B each): full[0..5], empty[0..5], acc_full[0..1], acc_empty[0..1]
  const uint32_t bar_full = bars, bar_empty = bars + 8 * k2Stages, bar_acc_full = bars + 16 * k2Stages,
                 bar_acc_empty = bars + 16 * k2Stages + 8 * kAccBufs;
  uint8_t* misc = base_ptr + k2Stages * k2StageBytes + 16 * k2Stages + 16 * kAccBufs;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
  float* bias_smem = reinterpret_cast<float*>(base_ptr + k2Stages * k2StageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster = static_cast<int>(cluster_id_x()), num_clusters = static_cast<int>(cluster_count_x());
  const int tiles_m2 = (p.M + 2 * kTileM - 1) / (2 * kTileM), tiles_n = (p.N + kTileN - 1) / kTileN;
  const int num_tiles = tiles_m2 * tiles_n;
  const int k_blocks = (p.K + kTileK - 1) / kTileK;
  const PairSchedule sched(num_tiles, num_clusters, p.tail_halves);

  const bool tl = g_gemm_timeline_on != 0 && blockIdx.x == 0;
  if (tl && threadIdx.x == 0) g_gemm_timeline[0] = global_ns();
  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);   // the leader's arrive.expect_tx; bytes of both CTAs complete it
      mbar_init(bar_empty + 8 * s, 1);  // one multicast commit from the leader's MMA thread
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 8);  // four epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTmemCols);
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before anybody signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  if (tl && threadIdx.x == 0) g_gemm_timeline[1] = global_ns();

  if (warp == 0) {
    // ---------------- TMA producer (each CTA loads its own halves; completion lands on the leader's barrier)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      unsigned long long waited = 0;
      bool first = true;
      const bool hint_a = (p.ab_hint & 5) != 0, hint_b = (p.ab_hint & 10) != 0;
      const uint64_t pol_a = (p.ab_hint & 1) ? l2_policy_evict_last() : l2_policy_evict_first();
      const uint64_t pol_b = (p.ab_hint & 2) ? l2_policy_evict_last() : l2_policy_evict_first();
      for (int w = cluster; w < sched.items && alive; w += num_clusters) {
        const PairItem it = sched.at(w);
        int tm, tn;
        pair_tile_coords(it.tile, tiles_m2, tiles_n, &tm, &tn, p.group_m);
        const int m0 = tm * 2 * kTileM + static_cast<int>(rank) * kTileM;
        const bool is_half = it.width != kTileN;
        const int b_cols = it.width / 2;  // B columns this CTA holds: 128, or 64 for a half tile
        const int nb0 = tn * kTileN + it.half * (kTileN / 2) + static_cast<int>(rank) * b_cols;
        const uint32_t stage_tx = static_cast<uint32_t>(k2AStageBytes + b_cols * kTileK * 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          const unsigned long long w0 = tl ? global_ns() : 0;
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1)) { alive = false; break; }
          if (tl) {
            waited += global_ns() - w0;
            if (first) { g_gemm_timeline[2] = global_ns(); first = false; }
          }
          const uint32_t full_leader = map_to_cta(bar_full + 8 * stage, 0);
          const uint32_t sa = base + stage * k2StageBytes, sb = sa + k2AStageBytes;
          const int k0 = kb * kTileK;
          if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * stage_tx);
          auto load_a = [&](uint32_t dst, int c0, int c1) {
            if (hint_a) tma_load_2d_pair_hint(dst, &tmap_a, c0, c1, full_leader, pol_a);
            else tma_load_2d_pair(dst, &tmap_a, c0, c1, full_leader);
          };
          // K-major B comes in one box of b_cols rows (the half tile has a tensor map of its own, box 64 x 64);
          // N-major B comes in 64 x 64 boxes from the same map, one or two of them
          const CUtensorMap* mb = (is_half && !p.b_mn_major) ? &tmap_b_half : &tmap_b;
          auto load_b = [&](uint32_t dst, int c0, int c1) {
            if (hint_b) tma_load_2d_pair_hint(dst, mb, c0, c1, full_leader, pol_b);
            else tma_load_2d_pair(dst, mb, c0, c1, full_leader);
          };
          if (p.a_mn_major) {
            load_a(sa, m0, k0);
            load_a(sa + kChunkBytes, m0 + 64, k0);
          } else {
            load_a(sa, k0, m0);
          }
          if (p.b_mn_major) {
            load_b(sb, nb0, k0);
            if (!is_half) load_b(sb + kChunkBytes, nb0 + 64, k0);
          } else {
            load_b(sb, k0, nb0);
          }
          if (++stage == k2Stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (tl) g_gemm_timeline[11] = waited;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer: the leader's elected lane drives both CTAs' tensor cores
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      const uint32_t a_step = p.a_mn_major ? (2 * 1024) >> 4 : (kUmmaK * 2) >> 4;
      const uint32_t b_step = p.b_mn_major ? (2 * 1024) >> 4 : (kUmmaK * 2) >> 4;
      unsigned long long wait_data = 0, wait_acc = 0;
      bool first = true, first_tile = true;
      for (int w = cluster; w < sched.items && alive; w += num_clusters) {
        const uint32_t idesc = sched.at(w).width == kTileN ? p.idesc : p.idesc_half;
        unsigned long long w0 = tl ? global_ns() : 0;
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, 2)) { alive = false; break; }
        if (tl) wait_acc += global_ns() - w0;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kTileN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          w0 = tl ? global_ns() : 0;
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3)) { alive = false; break; }
          if (tl) {
            wait_data += global_ns() - w0;
            if (first) { g_gemm_timeline[3] = global_ns(); first = false; }
          }
          tc_fence_after();
          const uint32_t sa = base + stage * k2StageBytes, sb = sa + k2AStageBytes;
          const uint64_t adesc = make_smem_desc(sa, p.a_mn_major);
          const uint64_t bdesc = make_smem_desc(sb, p.b_mn_major);
#pragma unroll
          for (int k = 0; k < kTileK / kUmmaK; ++k)
            umma_f16_pair(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(bar_empty + 8 * stage);  // frees the stage in both CTAs
          if (++stage == k2Stages) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
        umma_commit_pair(bar_acc_full + 8 * acc);   // accumulator halves complete in both CTAs
        if (tl && first_tile) { g_gemm_timeline[4] = global_ns(); first_tile = false; }
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
      if (tl) { g_gemm_timeline[9] = wait_data; g_gemm_timeline[10] = wait_acc; }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs): this CTA's 128 rows x 256 columns
    const int sub = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    const bool tle = tl && warp == 2 && lane == 0;
    unsigned long long e_wait = 0, e_busy = 0, e_tiles = 0;
    for (int w = cluster; w < sched.items && alive; w += num_clusters) {
      const PairItem it = sched.at(w);
      int tm, tn;
      pair_tile_coords(it.tile, tiles_m2, tiles_n, &tm, &tn, p.group_m);
      const int row = tm * 2 * kTileM + static_cast<int>(rank) * kTileM + sub * 32 + lane;
      const int n0 = tn * kTileN + it.half * (kTileN / 2);
      const int chunks = it.width / 32;
      const unsigned long long e0 = tle ? global_ns() : 0;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, 4))) { alive = false; break; }
      tc_fence_after();
      const unsigned long long e1 = tle ? global_ns() : 0;
      if (tle) {
        e_wait += e1 - e0;
        if (e_tiles == 0) g_gemm_timeline[5] = e1;
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(sub * 32) << 16) + acc * kTileN;
      float* bs = bias_smem + (warp - 2) * kTileN;
#pragma unroll 1
      for (int h = 0; h < chunks; ++h) {
        const int col = n0 + lane + 32 * h;
        bs[lane + 32 * h] = (p.bias_dtype != 0 && col < p.N) ? bias_at(p, col) : 0.0f;
      }
      __syncwarp();
#pragma unroll 1
      for (int c = 0; c < chunks; c += 2) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[64];
        const bool two = col0 + 32 < p.N;
        if (two) {
          tmem_ld_32x32_pair(taddr + c * 32, r);
        } else {
          tmem_ld_32x32(taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        }
        epilogue_chunk(p, row, col0, &r[0], bs + c * 32);
        if (two) epilogue_chunk(p, row, col0 + 32, &r[32], bs + c * 32 + 32);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_acc_empty + 8 * acc, 0));  // the leader's barrier counts both CTAs
      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      if (tle) {
        const unsigned long long e2 = global_ns();
        e_busy += e2 - e1;
        if (e_tiles == 0) g_gemm_timeline[6] = e2;
        g_gemm_timeline[7] = e2;
        ++e_tiles;
      }
    }
    if (tle) { g_gemm_timeline[12] = e_wait; g_gemm_timeline[13] = e_busy; g_gemm_timeline[14] = e_tiles; }
  }

  // ---------------- teardown: neither CTA may leave while its partner can still touch its shared or tensor memory
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(16384);
  }
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (tl && threadIdx.x == 0) g_gemm_timeline[8] = global_ns();
}

// ================================================================== fp32 on the tensor cores: 3xTF32
// C = A * B with fp32 operands at close to fp32 accuracy, using kind::tf32 MMAs. Every operand is first split into
// hi = tf32(x) and lo = tf32(x - hi) (both exactly representable in TF32, x = hi + lo up to 2^-22 |x|), written
// K-major into the workspace by tf32_split_kernel; the main loop then accumulates, per 8-wide k step,
// A_lo*B_hi + A_hi*B_lo + A_hi*B_hi into the same fp32 accumulator in tensor memory (small terms first; the
// dropped A_lo*B_lo term is below 2^-22 of the product). Same roles, barriers and epilogue as the 16-bit kernel;
// tile 128x128, k slab 32 (one 128-byte swizzle row of fp32), 3 stages of 4 x 16 KiB.
// The tensor core rounds its fp32 accumulator toward zero at every k step, an error that grows linearly with the
// number of steps accumulated in place. K is therefore cut into chunks of 256: each chunk accumulates from zero in
// one of four 128-column accumulators, and the epilogue warps add the chunk results in registers with ordinary
// round-to-nearest fp32 additions while the next chunks are already being multiplied.
constexpr int k3TileN = 128;
constexpr int k3TileK = 32;
constexpr int k3Stages = 3;
constexpr int k3TileBytes = kTileM * k3TileK * 4;            // 16 KiB: one operand part of one stage
constexpr int k3StageBytes = 4 * k3TileBytes;               // A_hi, A_lo, B_hi, B_lo
constexpr int k3AccBufs = 4;
constexpr int k3ChunkBlocks = 8;                            // k slabs per accumulation chunk: 8 x 32 = 256
constexpr int k3TmemCols = k3AccBufs * k3TileN;             // 512
constexpr size_t k3SmemBytes = 1024 + size_t(k3Stages) * k3StageBytes + 256 + 4 * k3TileN * sizeof(float);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// src(r, k) = src[r * r_stride + k * k_stride] for r < R, k < K  ->  hi/lo[r * Kp + k] (Kp >= K, pad untouched:
// the tensor maps are encoded with K columns, so the pad is never read). 32x32 tiles through shared memory make
// both the read (along whichever index has unit stride) and the write (along k) coalesced.
__global__ void __launch_bounds__(256)
    tf32_split_kernel(const float* __restrict__ src, int64_t r_stride, int64_t k_stride, int64_t R, int64_t K, int64_t Kp,
                      float* __restrict__ hi, float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 32, k0 = static_cast<int64_t>(blockIdx.x) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const bool k_fast = k_stride <= r_stride;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int a = ty + 8 * i;  // slow index within the tile
    const int64_t r = k_fast ? r0 + a : r0 + tx, k = k_fast ? k0 + tx : k0 + a;
    const float v = (r < R && k < K) ? src[r * r_stride + k * k_stride] : 0.0f;
    if (k_fast) tile[a][tx] = v; else tile[tx][a] = v;  // tile[r][k]
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rr = ty + 8 * i;
    const int64_t r = r0 + rr, k = k0 + tx;
    if (r < R && k < K) {
      const float v = tile[rr][tx];
      uint32_t h, l;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
      const float rest = v - __uint_as_float(h);
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
      hi[r * Kp + k] = __uint_as_float(h);
      lo[r * Kp + k] = __uint_as_float(l);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
    gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_ahi, const __grid_constant__ CUtensorMap tmap_alo,
                       const __grid_constant__ CUtensorMap tmap_bhi, const __grid_constant__ CUtensorMap tmap_blo,
                       const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t bars = base + k3Stages * k3StageBytes;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * k3Stages, bar_acc_full = bars + 16 * k3Stages,
                 bar_acc_empty = bars + 16 * k3Stages + 8 * k3AccBufs;
  uint8_t* misc = base_ptr + k3Stages * k3StageBytes + 16 * k3Stages + 16 * k3AccBufs;
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
  float* bias_smem = reinterpret_cast<float*>(base_ptr + k3Stages * k3StageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kTileM - 1) / kTileM, tiles_n = (p.N + k3TileN - 1) / k3TileN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + k3TileK - 1) / k3TileK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k3Stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < k3AccBufs; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), k3TmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {  // TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        const int m0 = tm * kTileM, n0 = tn * k3TileN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, 1)) { alive = false; break; }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t s0 = base + stage * k3StageBytes;
          const int k0 = kb * k3TileK;
          mbar_expect_tx(full, k3StageBytes);
          tma_load_2d(s0, &tmap_ahi, k0, m0, full);
          tma_load_2d(s0 + k3TileBytes, &tmap_alo, k0, m0, full);
          tma_load_2d(s0 + 2 * k3TileBytes, &tmap_bhi, k0, n0, full);
          tma_load_2d(s0 + 3 * k3TileBytes, &tmap_blo, k0, n0, full);
          if (++stage == k3Stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {  // MMA issuer
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      constexpr uint32_t kStep = (8 * 4) >> 4;  // one k step of 8 fp32 = 32 B, in descriptor units of 16 B
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        for (int kb0 = 0; kb0 < k_blocks && alive; kb0 += k3ChunkBlocks) {
          if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, 2)) { alive = false; break; }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + acc * k3TileN;
          const int kb1 = min(kb0 + k3ChunkBlocks, k_blocks);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, 3)) { alive = false; break; }
            tc_fence_after();
            const uint32_t s0 = base + stage * k3StageBytes;
            const uint64_t ahi = make_smem_desc(s0, 0), alo = make_smem_desc(s0 + k3TileBytes, 0);
            const uint64_t bhi = make_smem_desc(s0 + 2 * k3TileBytes, 0), blo = make_smem_desc(s0 + 3 * k3TileBytes, 0);
#pragma unroll
            for (int k = 0; k < k3TileK / 8; ++k) {
              umma_tf32(tmem_d, alo + k * kStep, bhi + k * kStep, p.idesc, (kb != kb0 || k != 0) ? 1u : 0u);
              umma_tf32(tmem_d, ahi + k * kStep, blo + k * kStep, p.idesc, 1u);
              umma_tf32(tmem_d, ahi + k * kStep, bhi + k * kStep, p.idesc, 1u);
            }
            umma_commit(bar_empty + 8 * stage);
            if (++stage == k3Stages) { stage = 0; phase ^= 1u; }
          }
          if (!alive) break;
          umma_commit(bar_acc_full + 8 * acc);  // this chunk's partial product is complete
          if (++acc == k3AccBufs) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    const int sub = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
      const int row = tm * kTileM + sub * 32 + lane;
      const int n0 = tn * k3TileN;
      float* bs = bias_smem + (warp - 2) * k3TileN;
#pragma unroll
      for (int h = 0; h < k3TileN / 32; ++h) {
        const int col = n0 + lane + 32 * h;
        bs[lane + 32 * h] = (p.bias_dtype != 0 && col < p.N) ? bias_at(p, col) : 0.0f;
      }
      __syncwarp();
      // Running sum of this thread's row over the chunks: 128 floats in registers (every index below is a
      // compile-time constant), added with round-to-nearest.
      float run[k3TileN];
      for (int kb0 = 0; kb0 < k_blocks; kb0 += k3ChunkBlocks) {
        if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, 4))) { alive = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(sub * 32) << 16) + acc * k3TileN;
#pragma unroll
        for (int c = 0; c < k3TileN / 64; ++c) {
          uint32_t r[64];
          tmem_ld_32x32_pair(taddr + c * 64, r);
          if (kb0 == 0) {
#pragma unroll
            for (int j = 0; j < 64; ++j) run[c * 64 + j] = __uint_as_float(r[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) run[c * 64 + j] += __uint_as_float(r[j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
        if (++acc == k3AccBufs) { acc = 0; acc_phase ^= 1u; }
      }
      if (!alive) break;
#pragma unroll
      for (int c = 0; c < k3TileN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 < p.N) epilogue_chunk(p, row, col0, reinterpret_cast<const uint32_t*>(&run[c * 32]), bs + c * 32);
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(16384);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, k3TmemCols);
  }
}

// ------------------------------------------------------------------ host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      sym = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// Operand with `inner` contiguous elements per line, `outer` lines `ld` elements apart.
bool encode_operand(CUtensorMap* map, const void* base, DType dt, int64_t inner, int64_t outer, int64_t ld,
                    uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  // a single line has no meaningful pitch; any 16-byte multiple that covers it satisfies the encoder
  const cuuint64_t pitch = outer == 1 ? ((static_cast<cuuint64_t>(inner) * 2 + 15) / 16) * 16 : static_cast<cuuint64_t>(ld) * 2;
  const cuuint64_t strides[1] = {pitch};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType t = dt == DType::kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(map, t, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 0 = K-major, 1 = MN-major, -1 = neither stride is 1 / alignment rules not met
int operand_major(const void* data, int64_t mn_stride, int64_t k_stride, int64_t mn, int64_t k) {
  if (!aligned_to(data, 16)) return -1;
  if (k_stride == 1 && (mn == 1 || (mn_stride * 2) % 16 == 0) && mn_stride >= k) return 0;
  if (mn_stride == 1 && (k == 1 || (k_stride * 2) % 16 == 0) && k_stride >= mn) return 1;
  return -1;
}

bool is16(DType t) { return t == DType::kF16 || t == DType::kBF16; }

}  // namespace

bool gemm_tcgen05_eligible(const GemmProblem& p) {
  if (!is16(p.A.dtype) || p.A.dtype != p.B.dtype) return false;
  if (p.C.dtype != p.A.dtype && p.C.dtype != DType::kF32) return false;
  if (p.bias && p.bias_dtype != DType::kF32 && p.bias_dtype != p.A.dtype) return false;
  if (p.C.cs != 1) return false;
  if (p.M > 0x7fffff00 || p.N > 0x7fffff00 || p.K > 0x7fffff00) return false;
  // A is [M,K]: rs walks M, cs walks K.  B is [K,N]: rs walks K, cs walks N.
  if (operand_major(p.A.data, p.A.rs, p.A.cs, p.M, p.K) < 0) return false;
  if (operand_major(p.B.data, p.B.cs, p.B.rs, p.N, p.K) < 0) return false;
  return encode_fn() != nullptr;
}

namespace {

struct GemmChoice {
  bool pair = false;  // CTA pairs on 256x256 tiles, else one CTA per 128 x tn tile
  int tn = 256;
  int splits = 1;     // > 1: split-K over that many CTAs per tile (single-CTA kernel only)
};

// Kernel and tile shape by a small cost model: (rounds of tiles over the SMs, or SM pairs) x (relative duration of
// one round). The weights are the measured round times of a long-K problem (K = 8192: 44 / 51 / 65 us for one CTA
// per 128x64 / 128x128 / 128x256 tile, 56 us for a CTA pair per 256x256 tile), normalised to the pair. A narrow tile
// is cheaper per round but needs more rounds once it stops fitting the machine: 256 x 8192 x 8192 takes 51 us as one
// round of 128x128 tiles and 89 us as two rounds of 128x64 tiles; 1024^3 is fastest as one round of 128x64 tiles.
//
// Split-K: a product with few tiles and a long K (a small batch against a large weight matrix) is bound by how many
// bytes of the large operand are in flight; with one tile per CTA a 128x64 tile keeps 64 KiB of it in its ring and
// most SMs of a wide-tile launch are idle. Such products run on 128x256 (or 128x128) tiles with K divided over up to
// 8 CTAs per tile, so that all SMs stream the large operand with most of their shared memory; the fp32 parts are
// added in split order by splitk_finish_kernel (deterministic). Considered only when it is predicted to win and each
// part keeps at least 8 k blocks.
// AICF_GEMM_CTA_GROUP=1|2, AICF_GEMM_TILE_N=256|128|64 and AICF_GEMM_SPLITK=<n> (0 or 1 = off) override the choice
// (tuning and tests). The environment is read at the first GEMM of the process, not on every launch;
// gemm_reload_env_overrides() reads it again (a test or a sweep that changes a setting inside one process).
struct GemmEnvOverrides {
  int cta_group = 0;  // 0 = no override
  int tile_n = 0;
  bool splitk_set = false;
  int splitk = 0;
  int group_m = 0;    // AICF_GEMM_GROUP_M: rasterisation group in 128-row tiles (0 = default)
  int c_stream = -1;  // AICF_GEMM_C_STREAM: 0 / 1 (-1 = default)
  int ab_hint = -1;   // AICF_GEMM_AB_HINT: bit mask, see GemmParams (-1 = default)
  int tail_halves = -1;  // AICF_GEMM_TAIL_HALVES: 0 / 1 (-1 = default, on)
};
GemmEnvOverrides read_gemm_env() {
  {
    GemmEnvOverrides e;
    if (const char* s = std::getenv("AICF_GEMM_CTA_GROUP")) e.cta_group = s[0] == '1' ? 1 : s[0] == '2' ? 2 : 0;
    if (const char* s = std::getenv("AICF_GEMM_TILE_N")) e.tile_n = std::atoi(s);
    if (const char* s = std::getenv("AICF_GEMM_SPLITK")) e.splitk_set = true, e.splitk = std::atoi(s);
    if (const char* s = std::getenv("AICF_GEMM_GROUP_M")) e.group_m = std::atoi(s);
    if (const char* s = std::getenv("AICF_GEMM_C_STREAM")) e.c_stream = std::atoi(s);
    if (const char* s = std::getenv("AICF_GEMM_AB_HINT")) e.ab_hint = std::atoi(s);
    if (const char* s = std::getenv("AICF_GEMM_TAIL_HALVES")) e.tail_halves = std::atoi(s);
    return e;
  }
}
// The current settings. A reload publishes a new object and leaves the old one allocated: a launch on another thread
// may still be reading it, and reloads happen a handful of times in a test run.
std::atomic<const GemmEnvOverrides*> g_gemm_env{nullptr};
const GemmEnvOverrides& gemm_env_overrides() {
  const GemmEnvOverrides* e = g_gemm_env.load(std::memory_order_acquire);
  if (e == nullptr) {
    const GemmEnvOverrides* fresh = new GemmEnvOverrides(read_gemm_env());
    if (g_gemm_env.compare_exchange_strong(e, fresh, std::memory_order_acq_rel)) return *fresh;
    delete fresh;  // another thread published first
  }
  return *e;
}

GemmChoice choose_gemm(const GemmProblem& p) {
  GemmChoice c;
  const int64_t sms = sm_count();
  const int64_t pair_slots = sms / 2 > 0 ? sms / 2 : 1;
  auto rounds = [](int64_t tiles, int64_t slots) { return (tiles + slots - 1) / slots; };
  auto single_tiles = [&](int64_t w) { return ((p.M + kTileM - 1) / kTileM) * ((p.N + w - 1) / w); };
  const int64_t pair_tiles_all = ((p.M + 2 * kTileM - 1) / (2 * kTileM)) * ((p.N + kTileN - 1) / kTileN);
  const double cost_pair = p.M > kTileM ? 1.00 * static_cast<double>(rounds(pair_tiles_all, pair_slots)) : 1e30;
  const double cost64 = 0.78 * static_cast<double>(rounds(single_tiles(64), sms));
  const double cost128 = 0.90 * static_cast<double>(rounds(single_tiles(128), sms));
  const double cost256 = 1.16 * static_cast<double>(rounds(single_tiles(256), sms));
  c.tn = cost64 <= cost128 && cost64 <= cost256 ? 64 : cost128 <= cost256 ? 128 : 256;
  double best = c.tn == 64 ? cost64 : c.tn == 128 ? cost128 : cost256;
  c.pair = cost_pair <= best;
  if (c.pair) best = cost_pair;

  const int64_t k_blocks = (p.K + kTileK - 1) / kTileK;
  auto split_for = [&](int64_t w) -> int {
    const int64_t t = single_tiles(w);
    int64_t s = sms / t;
    if (s > k_blocks / 8) s = k_blocks / 8;
    if (s > 8) s = 8;
    if (s < 2) return 1;
    const int64_t per = (k_blocks + s - 1) / s;
    return static_cast<int>((k_blocks + per - 1) / per);  // no empty part
  };
  // Measured on M x 8192 x 8192 (bf16): M = 16 / 64 / 128 take 33 / 38 / 44 us split four ways on 128x256 tiles
  // against 49 us unsplit (the pass that adds the parts costs 2-10 us, growing with M); at M = 256 (64 tiles) the
  // split is already slower than one round of 128x128 tiles. Hence: only when the widest tiles fill at most a quarter
  // of the SMs, and the widest tile whose parts occupy most of the machine.
  if (k_blocks >= 64 && !c.pair) {
    const int widths[3] = {256, 128, 64};
    int best_w = 0, best_s = 1;
    int64_t best_ctas = 0;
    for (int i = 0; i < 3; ++i) {
      const int64_t t = single_tiles(widths[i]);
      if (single_tiles(256) * 4 > sms) break;
      const int sp = split_for(widths[i]);
      if (sp < 2) continue;
      const int64_t ctas = t * sp;
      if (ctas > best_ctas) {
        best_ctas = ctas;
        best_w = widths[i];
        best_s = sp;
      }
      if (ctas * 10 >= sms * 7) break;  // this width already occupies 70 % of the SMs
    }
    // Same CTA count from tiles half as wide and half as many parts: the adding pass moves M x N x parts floats, so
    // past M = 64 fewer parts win (M = 128: 40.5 us as 128x128 tiles in 2 parts, 43.7 us as 128x256 tiles in 4; at
    // M = 16 the wide tile is ahead, 33.5 against 35.3 us).
    if (best_w == 256 && best_s >= 4 && best_s % 2 == 0 && p.M > 64 && single_tiles(128) == 2 * single_tiles(256)) {
      best_w = 128;
      best_s /= 2;
    }
    if (best_w != 0) {
      c.tn = best_w;
      c.splits = best_s;
    }
  }
  const GemmEnvOverrides& env = gemm_env_overrides();
  if (env.cta_group == 1) c.pair = false;
  if (env.cta_group == 2 && p.M > kTileM) c.pair = true, c.splits = 1;
  if (env.tile_n == 256 || env.tile_n == 128 || env.tile_n == 64) {
    if (env.tile_n != c.tn) c.splits = 1;
    c.tn = env.tile_n;
  }
  if (env.splitk_set) {
    int v = env.splitk;
    if (v <= 1) {
      c.splits = 1;
    } else if (!c.pair) {
      if (v > 8) v = 8;
      if (v > k_blocks) v = static_cast<int>(k_blocks);
      const int64_t per = (k_blocks + v - 1) / v;
      c.splits = static_cast<int>((k_blocks + per - 1) / per);
    }
  }
  if (c.pair) c.splits = 1;
  return c;
}

// result[m][n] = epilogue(sum over splits of partial[s][m][n]), parts added in split order. Four columns per thread
// (N % 4 == 0 is guaranteed by the caller: the parts are written with 16-byte stores).
__device__ __forceinline__ float splitk_mask_at(const GemmParams& p, int64_t moff) {
  if (p.c_dtype == static_cast<int>(DType::kF32)) return static_cast<const float*>(p.mask)[moff];
  if (p.c_dtype == static_cast<int>(DType::kBF16)) return __bfloat162float(static_cast<const __nv_bfloat16*>(p.mask)[moff]);
  return __half2float(static_cast<const __half*>(p.mask)[moff]);
}
__global__ void __launch_bounds__(256) splitk_finish_kernel(GemmParams p) {
  const int64_t total4 = static_cast<int64_t>(p.M) * p.N / 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int n4 = p.N / 4;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total4; i += stride) {
    const int row = static_cast<int>(i / n4), col = static_cast<int>(i % n4) * 4;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < p.splits; ++s) {
      const float4 t = __ldcs(reinterpret_cast<const float4*>(p.partial) + static_cast<int64_t>(s) * total4 + i);
      acc.x += t.x;
      acc.y += t.y;
      acc.z += t.z;
      acc.w += t.w;
    }
    float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (p.bias_dtype != 0) v[e] += bias_at(p, col + e);
      if (p.relu) v[e] = fmaxf(v[e], 0.0f);
      if (p.mask && !(splitk_mask_at(p, static_cast<int64_t>(row) * p.mask_ld + col + e) > 0.0f)) v[e] = 0.0f;
    }
    const int64_t off = static_cast<int64_t>(row) * p.ldc + col;
    if (p.c_dtype == static_cast<int>(DType::kF32)) {
      float* dst = static_cast<float*>(p.C) + off;
      if (p.c_vec_ok) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      else { dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; dst[3] = v[3]; }
    } else {
      uint2 w;
      if (p.c_dtype == static_cast<int>(DType::kBF16)) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        w.x = *reinterpret_cast<const uint32_t*>(&lo);
        w.y = *reinterpret_cast<const uint32_t*>(&hi);
      } else {
        const __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
        w.x = *reinterpret_cast<const uint32_t*>(&lo);
        w.y = *reinterpret_cast<const uint32_t*>(&hi);
      }
      uint16_t* dst = static_cast<uint16_t*>(p.C) + off;
      if (p.c_vec_ok) {
        *reinterpret_cast<uint2*>(dst) = w;  // rows are 16-byte aligned and col is a multiple of 4: 8-byte aligned
      } else {
        dst[0] = static_cast<uint16_t>(w.x & 0xFFFFu);
        dst[1] = static_cast<uint16_t>(w.x >> 16);
        dst[2] = static_cast<uint16_t>(w.y & 0xFFFFu);
        dst[3] = static_cast<uint16_t>(w.y >> 16);
      }
    }
  }
}

}  // namespace

// Bytes of workspace the 16-bit GEMM wants for this problem (0 unless it is split over K).
size_t gemm_tcgen05_workspace(const GemmProblem& p) {
  if (!gemm_tcgen05_eligible(p)) return 0;
  const GemmChoice c = choose_gemm(p);
  return c.splits > 1 ? static_cast<size_t>(c.splits) * static_cast<size_t>(p.M) * static_cast<size_t>(p.N) * sizeof(float) : 0;
}

Status gemm_tcgen05_run(const GemmProblem& p, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (!gemm_tcgen05_eligible(p)) return Status::NotImplemented;
  const int a_major = operand_major(p.A.data, p.A.rs, p.A.cs, p.M, p.K);
  const int b_major = operand_major(p.B.data, p.B.cs, p.B.rs, p.N, p.K);
  GemmChoice choice = choose_gemm(p);
  if (choice.splits > 1) {  // no (or too little) workspace: run unsplit rather than fail
    const size_t need = static_cast<size_t>(choice.splits) * static_cast<size_t>(p.M) * static_cast<size_t>(p.N) * sizeof(float);
    if (!ws || ws_bytes < need || !aligned_to(ws, 16) || p.N % 4 != 0) choice.splits = 1;
  }
  const bool pair = choice.pair;
  const int tn = choice.tn;
  CUtensorMap ta, tb;
  const uint32_t b_rows = pair ? k2HalfN : static_cast<uint32_t>(tn);
  bool ok_maps = a_major == 0 ? encode_operand(&ta, p.A.data, p.A.dtype, p.K, p.M, p.A.rs, kTileK, kTileM)
                              : encode_operand(&ta, p.A.data, p.A.dtype, p.M, p.K, p.A.cs, 64, kTileK);
  ok_maps = ok_maps && (b_major == 0 ? encode_operand(&tb, p.B.data, p.B.dtype, p.K, p.N, p.B.cs, kTileK, b_rows)
                                     : encode_operand(&tb, p.B.data, p.B.dtype, p.N, p.K, p.B.rs, 64, kTileK));
  if (!ok_maps) return Status::Internal;
  // the paired kernel's half tiles take K-major B in boxes of 64 rows
  CUtensorMap tb_half = tb;
  if (pair && b_major == 0 && !encode_operand(&tb_half, p.B.data, p.B.dtype, p.K, p.N, p.B.cs, kTileK, k2HalfN / 2))
    return Status::Internal;

  GemmParams g{};
  g.C = const_cast<void*>(p.C.data);
  g.bias = p.bias;
  g.ldc = p.C.rs;
  g.bias_stride = p.bias_stride;
  g.mask = p.mask;
  g.mask_ld = p.mask_ld;
  g.mask_vec_ok = p.mask ? (aligned_to(p.mask, 16) && ((p.mask_ld * dtype_size_bytes(p.C.dtype)) % 16 == 0)) : 0;
  g.M = static_cast<int>(p.M);
  g.N = static_cast<int>(p.N);
  g.K = static_cast<int>(p.K);
  g.c_dtype = static_cast<int>(p.C.dtype);
  g.bias_dtype = p.bias ? static_cast<int>(p.bias_dtype) : 0;
  g.relu = p.relu ? 1 : 0;
  g.a_mn_major = a_major;
  g.b_mn_major = b_major;
  const uint32_t fmt = p.A.dtype == DType::kBF16 ? 1u : 0u;
  // instruction descriptor: D=f32 (bits 4-5 = 1), A/B format (bits 7-9 / 10-12), A/B major (bits 15/16),
  // N>>3 (bits 17-22), M>>4 (bits 24-28)
  g.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(a_major) << 15) |
            (static_cast<uint32_t>(b_major) << 16) | (static_cast<uint32_t>((pair ? kTileN : tn) >> 3) << 17) |
            (static_cast<uint32_t>((pair ? 2 * kTileM : kTileM) >> 4) << 24);
  g.idesc_half = (g.idesc & ~(0x3Fu << 17)) | (static_cast<uint32_t>((kTileN / 2) >> 3) << 17);
  const int c_elem = dtype_size_bytes(p.C.dtype);
  g.c_vec_ok = aligned_to(p.C.data, 16) && ((p.C.rs * c_elem) % 16 == 0);
  g.splits = choice.splits;
  g.partial = choice.splits > 1 ? static_cast<float*>(ws) : nullptr;
  {
    const GemmEnvOverrides& env = gemm_env_overrides();
    g.group_m = env.group_m >= 2 ? env.group_m : kGroupM;
    g.c_stream = env.c_stream >= 0 ? (env.c_stream ? 1 : 0) : kDefaultCStream;
    g.ab_hint = env.ab_hint >= 0 ? (env.ab_hint & 15) : kDefaultAbHint;
    g.tail_halves = env.tail_halves >= 0 ? (env.tail_halves ? 1 : 0) : 1;
  }

  const int dev = device_slot();  // -1: a device beyond the per-device tables, set up again on every call
  cudaGetLastError();
  if (pair) {
    static std::atomic<int> max_clusters[kMaxDevices] = {};
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = k2SmemBytes;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int device_clusters = dev >= 0 ? max_clusters[dev].load(std::memory_order_acquire) : 0;
    if (device_clusters == 0) {
      if (cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(k2SmemBytes)) != cudaSuccess) {
        cudaGetLastError();
        return Status::Internal;
      }
      cfg.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_2cta_kernel, &cfg) != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = sm_count() / 2;
      }
      device_clusters = n;
      if (dev >= 0) max_clusters[dev].store(n, std::memory_order_release);
    }
    const int64_t pair_tiles = ((p.M + 2 * kTileM - 1) / (2 * kTileM)) * ((p.N + kTileN - 1) / kTileN);
    const int clusters = static_cast<int>(pair_tiles < device_clusters ? pair_tiles : device_clusters);
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_2cta_kernel, ta, tb, tb_half, g) != cudaSuccess) {
      cudaGetLastError();
      return Status::Internal;
    }
    return launch_status();
  }
  const int64_t tiles = ((p.M + kTileM - 1) / kTileM) * ((p.N + tn - 1) / tn) * choice.splits;
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  auto go = [&](auto tag) -> Status {
    constexpr int TN = decltype(tag)::value;
    static PerDeviceOnce smem_opt_in;
    if (!smem_opt_in.run([] {
          return cudaFuncSetAttribute(gemm_tcgen05_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(SingleCfg<TN>::kSmem)) == cudaSuccess;
        })) {
      cudaGetLastError();
      return Status::Internal;
    }
    gemm_tcgen05_kernel<TN><<<grid, kThreads, SingleCfg<TN>::kSmem, stream>>>(ta, tb, g);
    return launch_status();
  };
  const Status st = tn == 256 ? go(std::integral_constant<int, 256>{})
                              : tn == 128 ? go(std::integral_constant<int, 128>{}) : go(std::integral_constant<int, 64>{});
  if (st != Status::Ok || choice.splits <= 1) return st;
  const int64_t total4 = static_cast<int64_t>(p.M) * p.N / 4;
  splitk_finish_kernel<<<streaming_grid(total4, 256, kStreamBlocksPerSm), 256, 0, stream>>>(g);
  return launch_status();
}

// ------------------------------------------------------------------ 3xTF32 host side
namespace {

int64_t tf32_kp(int64_t K) { return (K + 3) / 4 * 4; }  // row pitch of the split operands: a multiple of 16 bytes

bool encode_f32_kmajor(CUtensorMap* map, const float* base, int64_t K, int64_t rows, int64_t Kp, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(Kp) * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(k3TileK), box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool gemm_tf32x3_eligible(const GemmProblem& p) {
  if (p.A.dtype != DType::kF32 || p.B.dtype != DType::kF32 || p.C.dtype != DType::kF32) return false;
  if (p.bias && p.bias_dtype != DType::kF32) return false;
  if (p.C.cs != 1) return false;
  if (p.M > 0x7fffff00 || p.N > 0x7fffff00 || p.K > 0x7fffff00) return false;
  return encode_fn() != nullptr;
}

// hi and lo copies of both operands, K-major: 2 * (M + N) * Kp floats, each part 1024-byte aligned.
size_t gemm_tf32x3_workspace(const GemmProblem& p) {
  const size_t kp = static_cast<size_t>(tf32_kp(p.K));
  auto part = [&](int64_t rows) { return (static_cast<size_t>(rows) * kp * 4 + 1023) / 1024 * 1024; };
  return 2 * part(p.M) + 2 * part(p.N) + 1024;
}

Status gemm_tf32x3_run(const GemmProblem& p, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (!gemm_tf32x3_eligible(p)) return Status::NotImplemented;
  const size_t need = gemm_tf32x3_workspace(p);
  if (!ws || ws_bytes < need) return Status::InvalidArgument;
  const int64_t kp = tf32_kp(p.K);
  auto part = [&](int64_t rows) { return (static_cast<size_t>(rows) * kp * 4 + 1023) / 1024 * 1024; };
  uint8_t* w = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ws) + 1023) & ~uintptr_t(1023));
  float* ahi = reinterpret_cast<float*>(w);
  float* alo = reinterpret_cast<float*>(w + part(p.M));
  float* bhi = reinterpret_cast<float*>(w + 2 * part(p.M));
  float* blo = reinterpret_cast<float*>(w + 2 * part(p.M) + part(p.N));

  cudaGetLastError();
  const dim3 ga(static_cast<unsigned>((p.K + 31) / 32), static_cast<unsigned>((p.M + 31) / 32));
  const dim3 gb(static_cast<unsigned>((p.K + 31) / 32), static_cast<unsigned>((p.N + 31) / 32));
  if (ga.y > 65535u || gb.y > 65535u) return Status::NotImplemented;
  // A is [M,K]: rs walks M, cs walks K.  B is [K,N]: rs walks K, cs walks N; its split copy is [N,K].
  tf32_split_kernel<<<ga, 256, 0, stream>>>(static_cast<const float*>(p.A.data), p.A.rs, p.A.cs, p.M, p.K, kp, ahi, alo);
  tf32_split_kernel<<<gb, 256, 0, stream>>>(static_cast<const float*>(p.B.data), p.B.cs, p.B.rs, p.N, p.K, kp, bhi, blo);
  if (launch_status() != Status::Ok) return Status::Internal;

  CUtensorMap mahi, malo, mbhi, mblo;
  if (!encode_f32_kmajor(&mahi, ahi, p.K, p.M, kp, kTileM) || !encode_f32_kmajor(&malo, alo, p.K, p.M, kp, kTileM) ||
      !encode_f32_kmajor(&mbhi, bhi, p.K, p.N, kp, k3TileN) || !encode_f32_kmajor(&mblo, blo, p.K, p.N, kp, k3TileN))
    return Status::Internal;

  GemmParams g{};
  g.C = const_cast<void*>(p.C.data);
  g.bias = p.bias;
  g.ldc = p.C.rs;
  g.bias_stride = p.bias_stride;
  g.mask = p.mask;
  g.mask_ld = p.mask_ld;
  g.mask_vec_ok = p.mask ? (aligned_to(p.mask, 16) && ((p.mask_ld * 4) % 16 == 0)) : 0;
  g.M = static_cast<int>(p.M);
  g.N = static_cast<int>(p.N);
  g.K = static_cast<int>(p.K);
  g.c_dtype = static_cast<int>(DType::kF32);
  g.bias_dtype = p.bias ? static_cast<int>(p.bias_dtype) : 0;
  g.relu = p.relu ? 1 : 0;
  // D = f32, A/B format TF32 (2), both K-major, N >> 3, M >> 4
  g.idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(k3TileN >> 3) << 17) |
            (static_cast<uint32_t>(kTileM >> 4) << 24);
  g.c_vec_ok = aligned_to(p.C.data, 16) && ((p.C.rs * 4) % 16 == 0);

  static PerDeviceOnce smem_opt_in;
  if (!smem_opt_in.run([] {
        return cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(k3SmemBytes)) == cudaSuccess;
      })) {
    cudaGetLastError();
    return Status::Internal;
  }
  const int64_t tiles = ((p.M + kTileM - 1) / kTileM) * ((p.N + k3TileN - 1) / k3TileN);
  const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
  gemm_tf32x3_kernel<<<grid, kThreads, k3SmemBytes, stream>>>(mahi, malo, mbhi, mblo, g);
  return launch_status();
}

void gemm_reload_env_overrides() {
  g_gemm_env.store(new GemmEnvOverrides(read_gemm_env()), std::memory_order_release);
}

// Reads (and optionally clears) the device status word written by a GEMM that gave up waiting.
// Synchronises the device: meant for tests and for a check after a step, not for the launch path.
int gemm_tcgen05_status(bool clear) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (clear && v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  }
  return v;
}

// Tuning aid: enable / disable the CTA-0 timeline and read its 16 slots (synchronises the device).
int gemm_tcgen05_timeline(int enable, unsigned long long* out16) {
  if (out16) {
    if (cudaMemcpyFromSymbol(out16, g_gemm_timeline, sizeof(unsigned long long) * 16) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
  }
  if (cudaMemcpyToSymbol(g_gemm_timeline_on, &enable, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return 0;
}

}  // namespace aicf::cuda
