#pragma once
// Building blocks of the row kernels (softmax, softmax cross-entropy, layer norm): a block owns one row at a
// time, keeps it in registers, and prefetches its next row into shared memory with one bulk asynchronous copy.
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

// ------------------------------------------------------------------ row pipeline plumbing
constexpr unsigned long long kRowWaitBudgetNs = 1000000000ull;  // a row copy that takes 1 s is lost

// Dynamic shared memory: [row buffer: row_bytes][mbarrier: 8 B]. Thread 0 drives the copies.
struct RowPipe {
  uint32_t buf, bar;
  uint32_t phase;
  __device__ __forceinline__ void init(uint8_t* smem, uint32_t row_bytes) {
    buf = sm100::smem_addr(smem);
    bar = buf + row_bytes;
    phase = 0;
    if (threadIdx.x == 0) {
      sm100::mbar_init(bar, 1);
      sm100::mbar_init_fence();
    }
    __syncthreads();
  }
  __device__ __forceinline__ void fetch(const void* row, uint32_t row_bytes) {  // thread 0 only
    sm100::mbar_expect_tx(bar, row_bytes);
    sm100::bulk_copy_g2s(buf, row, row_bytes, bar);
  }
  // Block-uniform: false when any thread's wait expired (the block then stops); *status_word is then set to 1.
  __device__ __forceinline__ bool arrived(int* status_word) {
    const bool ok = sm100::mbar_wait_bounded(bar, phase, kRowWaitBudgetNs);
    phase ^= 1u;
    if (__syncthreads_or(ok ? 0 : 1)) {
      if (threadIdx.x == 0) atomicExch(status_word, 1);
      return false;
    }
    return true;
  }
};

// threads/packets choice shared by softmax and softmax-CE
struct RowCfg {
  int threads = 0;
  int packets = 0;  // 0 -> fallback
};
// max_packets bounds the registers a thread spends on the row: 8 packets of fp32 or 4 packets of a
// 16-bit type are 32 floats after unpacking, which fits the 64-register budget of a 1024-thread block.
inline RowCfg pick_row_cfg(int64_t n_packets, int max_packets) {
  RowCfg c;
  int threads = 128;
  while (threads < 1024 && static_cast<int64_t>(threads) * 4 < n_packets) threads *= 2;
  const int64_t per = (n_packets + threads - 1) / threads;
  c.threads = threads;
  c.packets = per <= 1 ? 1 : per <= 2 ? 2 : per <= 4 ? 4 : per <= 8 ? 8 : 0;
  if (c.packets > max_packets) c.packets = 0;
  return c;
}

// Dynamic shared memory of the pipelined kernels: the row plus its mbarrier.
inline size_t row_pipe_smem(int64_t row_bytes) { return static_cast<size_t>(row_bytes) + 16; }
constexpr size_t kMaxRowPipeSmem = 200 * 1024;

// Resident blocks per SM given threads and shared memory per block (227 KiB usable, ~1 KiB reserved per block).
inline int row_pipe_blocks_per_sm(int threads, size_t smem) {
  int by_threads = 2048 / threads;
  int by_smem = static_cast<int>((227 * 1024) / (smem + 1024));
  int b = by_threads < by_smem ? by_threads : by_smem;
  return b < 1 ? 1 : (b > 16 ? 16 : b);
}

template <typename K>
bool allow_smem(K kernel, size_t smem) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess;
}

}  // namespace aicf::cuda::rowk
