#pragma once
// Building blocks of the row kernels (softmax, softmax cross-entropy, layer norm): a block owns one row at a
// time, keeps it in registers, and prefetches its next row into shared memory with one bulk asynchronous copy.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "sm100_async.cuh"

namespace aicf::cuda::rowk {

constexpr int kMaxWarps = 32;

// Block-wide max / sum. Every thread returns the same value. Warp partials go through shared memory and are
// folded by the first warp with a fixed shuffle tree (a 1024-thread block would otherwise spend more time on
// every thread re-reading 32 partials than on the row itself).
template <bool kIsMax>
__device__ __forceinline__ float block_reduce(float v, float* smem /*[kMaxWarps + 1]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = kIsMax ? warp_max(v) : warp_sum(v);
  __syncthreads();  // smem may still be read by the previous reduction
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float r = lane < nwarps ? smem[lane] : (kIsMax ? -INFINITY : 0.0f);
    r = kIsMax ? warp_max(r) : warp_sum(r);
    if (lane == 0) smem[kMaxWarps] = r;
  }
  __syncthreads();
  return smem[kMaxWarps];
}

// The same reduction with two barriers instead of three: nothing guards `area` against the previous call, so
// consecutive calls in a block must alternate between two areas (a thread still reading the total of call i is then
// never overtaken by the partial writes of call i + 1, and call i + 2 is two barriers later). Everything a thread did
// before the call (its shared-memory reads of the current row in particular) is ordered before the first barrier.
template <bool kIsMax>
__device__ __forceinline__ float block_reduce_2b(float v, float* area /*[kMaxWarps + 1]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = kIsMax ? warp_max(v) : warp_sum(v);
  if (lane == 0) area[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float r = lane < nwarps ? area[lane] : (kIsMax ? -INFINITY : 0.0f);
    r = kIsMax ? warp_max(r) : warp_sum(r);
    if (lane == 0) area[kMaxWarps] = r;
  }
  __syncthreads();
  return area[kMaxWarps];
}

// ------------------------------------------------------------------ row pipeline plumbing
constexpr unsigned long long kRowWaitBudgetNs = 1000000000ull;  // a row copy that takes 1 s is lost

// Dynamic shared memory: [row buffer: row_bytes][mbarrier: 8 B]. Thread 0 drives the copies.
struct RowPipe {
  uint32_t buf, bar;
  uint32_t phase;
  __device__ __forceinline__ void init(uint8_t* smem, uint32_t row_bytes, int* failed_flag) {
    buf = sm100::smem_addr(smem);
    bar = buf + row_bytes;
    phase = 0;
    if (threadIdx.x == 0) {
      sm100::mbar_init(bar, 1);
      sm100::mbar_init_fence();
      *failed_flag = 0;
    }
    __syncthreads();
  }
  __device__ __forceinline__ void fetch(const void* row, uint32_t row_bytes) {  // thread 0 only
    sm100::mbar_expect_tx(bar, row_bytes);
    sm100::bulk_copy_g2s(buf, row, row_bytes, bar);
  }
  // Block-uniform wait with a barrier of its own: false when any thread's wait expired (the block then stops).
  __device__ __forceinline__ bool arrived(int* status_word) {
    const bool ok = sm100::mbar_wait_bounded(bar, phase, kRowWaitBudgetNs);
    phase ^= 1u;
    if (__syncthreads_or(ok ? 0 : 1)) {
      if (threadIdx.x == 0) atomicExch(status_word, 1);
      return false;
    }
    return true;
  }
  // Waits for the row without a barrier. A wait that runs out sets *failed_flag (shared memory, zeroed before the
  // loop); the caller tests the flag after the next block-wide barrier, where every thread sees the same value, and
  // leaves the loop there. Until then the threads work on whatever the buffer holds, which is harmless.
  __device__ __forceinline__ void wait_row(int* failed_flag) {
    if (!sm100::mbar_wait_bounded(bar, phase, kRowWaitBudgetNs)) *failed_flag = 1;
    phase ^= 1u;
  }
};

// threads/packets choice shared by softmax and softmax-CE
struct RowCfg {
  int threads = 0;
  int packets = 0;  // 0 -> fallback
};
// max_packets bounds the registers a thread spends on the row: 8 packets of fp32 or 4 packets of a
// 16-bit type are 32 floats after unpacking, which fits the 64-register budget of a 1024-thread block.
// Blocks start at one warp and grow only while a thread would hold more than four packets: a narrow row is then a
// warp's job (its "block" barriers cost nothing and up to 32 such blocks share an SM) instead of leaving most of a
// 128-thread block idle. Measured on [65536,1024]: bf16 softmax 0.65 -> 0.91 of the copy rate, f32 0.86 -> 0.94,
// f32 cross-entropy 0.74 -> 0.91; on [262144,256] f32 softmax 0.51 -> 0.92.
inline RowCfg pick_row_cfg(int64_t n_packets, int max_packets) {
  RowCfg c;
  // AICF_ROW_PACKETS=n (tuning, read once per process): packets a thread may hold before the block grows (default 4)
  static const int per_thread = [] {
    const char* e = std::getenv("AICF_ROW_PACKETS");
    const int v = e ? std::atoi(e) : 0;
    return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 4;
  }();
  const int grow_at = per_thread < max_packets ? per_thread : max_packets;
  int threads = 32;
  while (threads < 1024 && static_cast<int64_t>(threads) * grow_at < n_packets) threads *= 2;
  const int64_t per = (n_packets + threads - 1) / threads;
  c.threads = threads;
  c.packets = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : per <= 8 ? 8 : 0;
  if (c.packets > max_packets) c.packets = 0;
  return c;
}

// Dynamic shared memory of the pipelined kernels: the row plus its mbarrier.
inline size_t row_pipe_smem(int64_t row_bytes) {
  // AICF_ROW_SMEM_PAD (tuning, read once per process): unused bytes added to every block's shared memory, to bound how
  // many blocks an SM holds
  static const size_t pad = [] {
    const char* e = std::getenv("AICF_ROW_SMEM_PAD");
    const long v = e ? std::atol(e) : 0;
    return static_cast<size_t>(v > 0 ? (v / 16) * 16 : 0);
  }();
  return static_cast<size_t>(row_bytes) + 16 + pad;
}
constexpr size_t kMaxRowPipeSmem = 200 * 1024;

// Resident blocks per SM given threads and shared memory per block (227 KiB usable, ~1 KiB reserved per block).
inline int row_pipe_blocks_per_sm(int threads, size_t smem) {
  int by_threads = 2048 / threads;
  int by_smem = static_cast<int>((227 * 1024) / (smem + 1024));
  int b = by_threads < by_smem ? by_threads : by_smem;
  return b < 1 ? 1 : (b > 32 ? 32 : b);
}

// Whether a row that fills every thread's packets exactly takes the kernel variant without per-packet range checks.
// AICF_ROW_FULL (tuning, read once per process): 0 = never, 1 = always, unset = by element size (see use_full_rows).
inline int row_full_override() {
  static const int v = [] {
    const char* e = std::getenv("AICF_ROW_FULL");
    return (e == nullptr || e[0] == 0) ? -1 : (e[0] == '0' ? 0 : 1);
  }();
  return v;
}
inline bool use_full_rows(bool exact_fit, size_t elem_bytes) {
  if (!exact_fit) return false;
  const int o = row_full_override();
  if (o >= 0) return o != 0;
  return elem_bytes < 4;
}
// Type of a thread's packet index. The 16-bit kernels are bound by instruction issue: 32-bit indices and no range
// checks took a quarter of their instructions away (layer norm [32768,4096] bf16: forward 5650 -> 6258 GB/s, backward
// 5392 -> 6035). The fp32 kernels are bound by HBM and measured slower with the leaner code (layer norm backward f32
// 6739 -> 5800 GB/s, softmax f32 6239 -> 5953): there the timing of the loads and stores decides, not the instruction
// count, so they keep the 64-bit index arithmetic and the checks they were tuned with.
template <typename T>
struct RowIdx {
  using type = std::conditional_t<sizeof(T) == 4, int64_t, int>;
};

template <typename K>
bool allow_smem(K kernel, size_t smem) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess;
}

// Shared memory to ask for so that an SM holds at most 1024 threads of a softmax / cross-entropy kernel (blocks of 128
// threads and more). These kernels read nothing through L1, so the unused bytes cost nothing, and fewer, equally long
// row streams per SM measured faster than filling the SM: softmax f32 [32768,4096] 6064 -> 6620 GB/s with four instead
// of five 256-thread blocks resident (whatever the grid: 4, 8, 12 or 16 blocks per SM), [32768,2048] 6214 -> 6473, bf16
// [32768,4096] 6387 -> 6473, cross-entropy f32 on 1024 columns 6377 -> 6489; three resident blocks lose again (6023), and
// 64-thread softmax blocks lose from the cap (6112 -> 5924), hence the threshold. The grid keeps its size. Layer norm
// reads gamma and beta through L1 and sits at 1024 threads per SM by its registers anyway: it does not use this.
inline size_t row_smem_capped_residency(size_t smem, int threads) {
  if (threads < 128) return smem;
  const size_t blocks = static_cast<size_t>(1024 / threads);
  const size_t want = (227 * 1024) / (blocks + 1) + 16;  // more than this and blocks + 1 no longer fit
  const size_t aligned = (want + 15) / 16 * 16;
  return aligned > smem ? aligned : smem;
}

// Blocks per SM the grid-stride row kernels are launched with. The default is the estimate above, which ignores
// registers and therefore over-subscribes some shapes (a 256-thread block at 46 registers fits five times, not
// eight): measured on [32768,4096] and [65536,1024], a grid of exactly the resident blocks was slower than the
// over-subscribed one (bf16 softmax 5736 against 6425 GB/s, f32 cross-entropy on 1024 columns 5679 against 6376),
// because blocks that start late run out of step with the first wave and smooth its read-then-write bursts.
// AICF_ROW_BLOCKS_PER_SM (tuning, read once per process): a number forces that many, "occ" asks the runtime for the
// resident count of this kernel at this block size and shared memory.
template <typename K>
int row_blocks_per_sm(K kernel, int threads, size_t smem) {
  static const int forced = [] {
    const char* e = std::getenv("AICF_ROW_BLOCKS_PER_SM");
    if (e == nullptr || e[0] == 0) return 0;
    if (e[0] == 'o') return -1;
    const int v = std::atoi(e);
    return v < 1 ? 0 : (v > 4096 ? 4096 : v);
  }();
  if (forced > 0) return forced;
  if (forced == 0) return row_pipe_blocks_per_sm(threads, smem);
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess || n < 1) {
    cudaGetLastError();
    return row_pipe_blocks_per_sm(threads, smem);
  }
  return n > 32 ? 32 : n;
}

}  // namespace aicf::cuda::rowk
