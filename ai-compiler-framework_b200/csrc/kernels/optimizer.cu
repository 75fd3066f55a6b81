// Optimizer-state kernels: fused Adam (two contracts), device step counter, device
// bias-correction scalars, SGD.
//
// Everything here is HBM-bound streaming work: 128-bit loads/stores with evict-first hints,
// 64-bit indexing, and a grid as large as the array needs at two packets per thread (up to
// kStreamBlocksPerSm blocks per SM, a grid-stride loop past that), so one launch covers any size
// (the reference caps its grid at 65535 blocks of scalar accesses).
#include <cstdlib>

#include "adam_math.cuh"
#include "common.cuh"

namespace aicf::cuda {

namespace {

bool f32_contig_rank1p(const TensorDesc& d) { return d.dtype == DType::kF32 && d.contiguous && d.rank() >= 1; }
bool f32_scalar0(const TensorDesc& d) { return d.dtype == DType::kF32 && d.rank() == 0 && d.contiguous; }
bool same_ptr(const TensorDesc& a, const TensorDesc& b) { return a.data == b.data; }

int64_t numel_raw(const TensorDesc& d) {
  int64_t n = 1;
  for (int i = 0; i < d.rank(); ++i) n *= d.shape[i];
  return n;
}

// Aliasing rules of the reference (ops/adam_step/launcher.cu:98-128): each of P/M/V may be updated
// in place; the gradient aliases nothing; no cross aliasing between the P, M and V groups.
bool adam_alias_violation(const TensorDesc& P, const TensorDesc& G, const TensorDesc& M, const TensorDesc& V,
                          const TensorDesc& Po, const TensorDesc& Mo, const TensorDesc& Vo) {
  const TensorDesc* others[] = {&P, &M, &V, &Po, &Mo, &Vo};
  for (const TensorDesc* o : others)
    if (same_ptr(G, *o)) return true;
  if (!same_ptr(Po, P) && (same_ptr(Po, M) || same_ptr(Po, V) || same_ptr(Po, Mo) || same_ptr(Po, Vo))) return true;
  if (!same_ptr(Mo, M) && (same_ptr(Mo, P) || same_ptr(Mo, V) || same_ptr(Mo, Po) || same_ptr(Mo, Vo))) return true;
  if (!same_ptr(Vo, V) && (same_ptr(Vo, P) || same_ptr(Vo, M) || same_ptr(Vo, Po) || same_ptr(Vo, Mo))) return true;
  return same_ptr(M, V) || same_ptr(P, M) || same_ptr(P, V);
}

// ----------------------------------------------------------------------------------------------
// One kernel template serves both contracts:
//   kDivisorScalars = true : bias corrections are two device scalars used as divisors
//                            (adam_step_f32_v0; reference kernel ops/adam_step/launcher.cu:257-293)
//   kDivisorScalars = false: the int32 step counter is read and 1-beta^t formed in the kernel;
//                            optional weight decay, optional 16-bit copy of the new parameter.
// ----------------------------------------------------------------------------------------------
struct AdamArgs {
  const float* p;
  const float* g;
  const float* m;
  const float* v;
  float* p_out;
  float* m_out;
  float* v_out;
  void* p_lp;             // optional 16-bit working copy of the new parameter (bf16 or f16)
  const float* bc1;       // divisor scalars (v0 contract)
  const float* bc2;
  const int32_t* step;    // step counter (fused contract)
  int64_t n;
  int64_t nvec;           // number of leading 4-element packets handled with 128-bit accesses
  AdamHyper h;
};

template <bool kDivisorScalars, int kLp>
__global__ void __launch_bounds__(256) adam_kernel(AdamArgs a) {
  float d1, d2;
  if (kDivisorScalars) {
    d1 = a.bc1[0];
    d2 = a.bc2[0];
  } else {
    adam_inverse_corrections(a.h, a.step[0], d1, d2);  // multipliers in the fused contract (see adam_one)
  }
  using V4 = Pack16<float>;
  const V4* P = reinterpret_cast<const V4*>(a.p);
  const V4* G = reinterpret_cast<const V4*>(a.g);
  const V4* M = reinterpret_cast<const V4*>(a.m);
  const V4* V = reinterpret_cast<const V4*>(a.v);
  V4* Po = reinterpret_cast<V4*>(a.p_out);
  V4* Mo = reinterpret_cast<V4*>(a.m_out);
  V4* Vo = reinterpret_cast<V4*>(a.v_out);

  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;

  // Two packets per stream per trip: 8 independent 16-byte loads in flight per thread.
  int64_t i = tid;
  for (; i + stride < a.nvec; i += 2 * stride) {
    V4 p[2], g[2], m[2], v[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t j = i + u * stride;
      p[u] = ld_stream(P + j);
      g[u] = ld_stream(G + j);
      m[u] = ld_stream(M + j);
      v[u] = ld_stream(V + j);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t j = i + u * stride;
      V4 po, mo, vo;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        adam_one<kDivisorScalars>(p[u].v[e], g[u].v[e], m[u].v[e], v[u].v[e], a.h, d1, d2, po.v[e], mo.v[e], vo.v[e]);
      st_stream(Mo + j, mo);
      st_stream(Vo + j, vo);
      st_stream(Po + j, po);
      if (kLp) store_lp_x4<kLp>(a.p_lp, j, po);
    }
  }
  for (; i < a.nvec; i += stride) {
    const V4 p = ld_stream(P + i), g = ld_stream(G + i), m = ld_stream(M + i), v = ld_stream(V + i);
    V4 po, mo, vo;
#pragma unroll
    for (int e = 0; e < 4; ++e)
      adam_one<kDivisorScalars>(p.v[e], g.v[e], m.v[e], v.v[e], a.h, d1, d2, po.v[e], mo.v[e], vo.v[e]);
    st_stream(Mo + i, mo);
    st_stream(Vo + i, vo);
    st_stream(Po + i, po);
    if (kLp) store_lp_x4<kLp>(a.p_lp, i, po);
  }
  // elements not covered by packets: the n % 4 tail, or everything when a buffer is not 16-byte aligned
  for (int64_t k = (a.nvec << 2) + tid; k < a.n; k += stride) {
    float po, mo, vo;
    adam_one<kDivisorScalars>(a.p[k], a.g[k], a.m[k], a.v[k], a.h, d1, d2, po, mo, vo);
    a.m_out[k] = mo;
    a.v_out[k] = vo;
    a.p_out[k] = po;
    if (kLp) store_lp_x1<kLp>(a.p_lp, k, po);
  }
}

// ---- grid of the streaming Adam kernels ----------------------------------------------------------------------------
// Every thread takes two 16-byte packets per array and the grid is as large as the array needs, up to kAdamBlocksPerSm
// blocks per SM: far more blocks than an SM holds at once. Measured on 2^28 elements (7.5 GB moved per launch), GB/s by
// blocks of 256 threads per SM: 4 (all resident, a long grid-stride loop each) 5983, 8 6171, 16 6321, 32 6421, 64 6522,
// 128 6615, 256 6761, 512 6857, 768 6919, 1024 (no loop left) 6911; a plain copy-like probe with the same four reads and
// three writes follows the same curve (6473 at 32, 6920 at 1024). A kernel that kept a ring of 16 KiB bulk copies per SM
// in flight instead (one persistent block per SM) reached 6277 and was dropped.
constexpr int kAdamThreads = 256;
constexpr int kAdamBlocksPerSm = kStreamBlocksPerSm;

template <bool kDiv, int kLp>
Status launch_adam(AdamArgs a, cudaStream_t stream) {
  if (a.n <= 0) return Status::Ok;
  const void* ptrs[] = {a.p, a.g, a.m, a.v, a.p_out, a.m_out, a.v_out};
  bool vec_ok = true;
  for (const void* q : ptrs) vec_ok = vec_ok && aligned_to(q, 16);
  if (kLp) vec_ok = vec_ok && aligned_to(a.p_lp, 8);
  // AICF_ADAM_GRID=n (tuning, read once per process): blocks per SM instead of kAdamBlocksPerSm
  static const int blocks_per_sm = [] {
    const char* e = std::getenv("AICF_ADAM_GRID");
    const int v = e ? std::atoi(e) : 0;
    return v >= 1 && v <= 1024 ? v : kAdamBlocksPerSm;
  }();
  a.nvec = vec_ok ? (a.n >> 2) : 0;
  const int64_t items = vec_ok ? (a.nvec / 2 + 1) : a.n;
  const int grid = streaming_grid(items, kAdamThreads, blocks_per_sm);
  cudaGetLastError();
  adam_kernel<kDiv, kLp><<<grid, kAdamThreads, 0, stream>>>(a);
  return launch_status();
}

// ---------------------------------------------------------------- adam_step_f32_v0 (reference contract)
// inputs [P,G,M,V,BC1,BC2] -> outputs [Pout,Mout,Vout]; BC1/BC2 are rank-0 f32 divisors.
bool adam_v0_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 6 || no != 3) return false;
  for (int i = 0; i < 4; ++i)
    if (!f32_contig_rank1p(in[i])) return false;
  for (int i = 0; i < 3; ++i)
    if (!f32_contig_rank1p(out[i])) return false;
  if (!f32_scalar0(in[4]) || !f32_scalar0(in[5])) return false;
  if (!same_shape(in[0], in[1]) || !same_shape(in[0], in[2]) || !same_shape(in[0], in[3])) return false;
  if (!same_shape(in[0], out[0]) || !same_shape(in[2], out[1]) || !same_shape(in[3], out[2])) return false;
  return !adam_alias_violation(in[0], in[1], in[2], in[3], out[0], out[1], out[2]);
}
bool adam_v0_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return adam_v0_check(in, ni, out, no);
}
Status adam_v0_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                      cudaStream_t stream) {
  if (!adam_v0_check(in, ni, out, no) || !attr) return Status::InvalidArgument;
  AdamArgs a{};
  a.p = static_cast<const float*>(in[0].data);  // out-of-place needs no staging copy: p is read, p_out written
  a.g = static_cast<const float*>(in[1].data);
  a.m = static_cast<const float*>(in[2].data);
  a.v = static_cast<const float*>(in[3].data);
  a.bc1 = static_cast<const float*>(in[4].data);
  a.bc2 = static_cast<const float*>(in[5].data);
  a.p_out = static_cast<float*>(out[0].data);
  a.m_out = static_cast<float*>(out[1].data);
  a.v_out = static_cast<float*>(out[2].data);
  a.n = numel_raw(in[0]);
  a.h = read_adam(attr);
  a.h.weight_decay = 0.0f;  // the v0 contract has no decay term
  return launch_adam<true, 0>(a, stream);
}
size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }

// ---------------------------------------------------------------- adam_step_f32_fused_v1
// inputs [P,G,M,V,step(i32 scalar)] -> outputs [P,M,V] or [P,M,V,P_lp (bf16|f16 copy)]; textbook Adam with
// bias correction 1-beta^t computed from the device step counter (t clamped to >= 1).
bool i32_scalar(const TensorDesc& d) {
  return d.dtype == DType::kI32 && (d.rank() == 0 || (d.rank() == 1 && d.shape[0] == 1));
}
bool adam_v1_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 5 || (no != 3 && no != 4)) return false;
  for (int i = 0; i < 4; ++i)
    if (!f32_contig_rank1p(in[i])) return false;
  for (int i = 0; i < 3; ++i)
    if (!f32_contig_rank1p(out[i])) return false;
  if (!i32_scalar(in[4])) return false;
  if (!same_shape(in[0], in[1]) || !same_shape(in[0], in[2]) || !same_shape(in[0], in[3])) return false;
  if (!same_shape(in[0], out[0]) || !same_shape(in[2], out[1]) || !same_shape(in[3], out[2])) return false;
  if (no == 4) {
    if ((out[3].dtype != DType::kBF16 && out[3].dtype != DType::kF16) || !out[3].contiguous || !same_shape(in[0], out[3]))
      return false;
    for (int i = 0; i < 4; ++i)
      if (same_ptr(out[3], in[i])) return false;
  }
  return !adam_alias_violation(in[0], in[1], in[2], in[3], out[0], out[1], out[2]);
}
bool adam_v1_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return adam_v1_check(in, ni, out, no);
}
Status adam_v1_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                      cudaStream_t stream) {
  if (!adam_v1_check(in, ni, out, no) || !attr) return Status::InvalidArgument;
  AdamArgs a{};
  a.p = static_cast<const float*>(in[0].data);
  a.g = static_cast<const float*>(in[1].data);
  a.m = static_cast<const float*>(in[2].data);
  a.v = static_cast<const float*>(in[3].data);
  a.step = static_cast<const int32_t*>(in[4].data);
  a.p_out = static_cast<float*>(out[0].data);
  a.m_out = static_cast<float*>(out[1].data);
  a.v_out = static_cast<float*>(out[2].data);
  a.p_lp = no == 4 ? out[3].data : nullptr;
  a.n = numel_raw(in[0]);
  a.h = read_adam(attr);
  if (no != 4) return launch_adam<false, 0>(a, stream);
  return out[3].dtype == DType::kBF16 ? launch_adam<false, 1>(a, stream) : launch_adam<false, 2>(a, stream);
}

// ---------------------------------------------------------------- adam_step_f32_multi_v1
// One launch for the whole optimizer step of a model: up to kMultiMax parameter tensors, each updated in place with
// the fused contract above. inputs [P0,G0,M0,V0, P1,G1,M1,V1, ..., step(i32 scalar)] -> outputs, per tensor,
// [Pt,Mt,Vt] followed by the tensor's 16-bit working copy when bit t of `lp_mask` is set. 'ADAM' payload
// <ffff fI> + <II> tensor count, lp_mask. The reference launches one kernel per tensor
// (ops/adam_step/launcher.cu:188-243); a plan is free to batch them: a model's biases and small matrices are
// launch-bound on their own and cannot fill the machine, and ten tails of ten grids add up.
//
// The grid walks one list of 8 KiB chunks over all tensors (a block per chunk: two packets per thread and array, the
// shape of adam_kernel, and as many blocks as there are chunks up to kAdamBlocksPerSm per SM); what is left of each
// tensor past its whole chunks (and tensors smaller than a chunk) is finished by one block per tensor.
constexpr int kMultiMax = 16;
constexpr int kMultiPackets = 2;                                  // 16-byte packets per thread per array per chunk
constexpr int kMultiChunk = kAdamThreads * kMultiPackets * 4;     // floats per array per chunk
struct AdamMultiArgs {
  float* p[kMultiMax];
  const float* g[kMultiMax];
  float* m[kMultiMax];
  float* v[kMultiMax];
  void* lp[kMultiMax];             // nullptr = no working copy
  int64_t n[kMultiMax];
  int64_t chunk_begin[kMultiMax + 1];  // whole chunks of tensors [0, t) come before tensor t's
  int lp_kind[kMultiMax];          // 0 none, 1 bf16, 2 f16
  int count;
  const int32_t* step;
  AdamHyper h;
};

__device__ __forceinline__ void adam_multi_store(const AdamMultiArgs& a, int t, int64_t packet, const Pack16<float>& po,
                                                 const Pack16<float>& mo, const Pack16<float>& vo) {
  using V4 = Pack16<float>;
  st_stream(reinterpret_cast<V4*>(a.m[t]) + packet, mo);
  st_stream(reinterpret_cast<V4*>(a.v[t]) + packet, vo);
  st_stream(reinterpret_cast<V4*>(a.p[t]) + packet, po);
  if (a.lp_kind[t] == 1) store_lp_x4<1>(a.lp[t], packet, po);
  if (a.lp_kind[t] == 2) store_lp_x4<2>(a.lp[t], packet, po);
}

__global__ void __launch_bounds__(kAdamThreads) adam_multi_kernel(const AdamMultiArgs a) {
  float d1, d2;
  adam_inverse_corrections(a.h, a.step[0], d1, d2);
  using V4 = Pack16<float>;
  const int64_t nchunks = a.chunk_begin[a.count];
  auto tensor_of = [&](int64_t chunk) {  // the tensor whose chunk range holds `chunk` (at most kMultiMax steps)
    int t = 0;
    while (t + 1 < a.count && chunk >= a.chunk_begin[t + 1]) ++t;
    return t;
  };
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int t = tensor_of(c);
    const int64_t base = (c - a.chunk_begin[t]) * (kMultiChunk / 4) + threadIdx.x;
    const V4* P = reinterpret_cast<const V4*>(a.p[t]);
    const V4* G = reinterpret_cast<const V4*>(a.g[t]);
    const V4* M = reinterpret_cast<const V4*>(a.m[t]);
    const V4* V = reinterpret_cast<const V4*>(a.v[t]);
    V4 p[kMultiPackets], g[kMultiPackets], m[kMultiPackets], v[kMultiPackets];
#pragma unroll
    for (int u = 0; u < kMultiPackets; ++u) {
      const int64_t j = base + u * kAdamThreads;
      p[u] = ld_stream(P + j);
      g[u] = ld_stream(G + j);
      m[u] = ld_stream(M + j);
      v[u] = ld_stream(V + j);
    }
#pragma unroll
    for (int u = 0; u < kMultiPackets; ++u) {
      V4 po, mo, vo;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        adam_one<false>(p[u].v[e], g[u].v[e], m[u].v[e], v[u].v[e], a.h, d1, d2, po.v[e], mo.v[e], vo.v[e]);
      adam_multi_store(a, t, base + u * kAdamThreads, po, mo, vo);
    }
  }
  // what the whole chunks leave over, one block per tensor
  for (int t = blockIdx.x; t < a.count; t += gridDim.x) {
    const int64_t done = (a.chunk_begin[t + 1] - a.chunk_begin[t]) * kMultiChunk;
    const int64_t left = a.n[t] - done;
    const int64_t pk0 = done >> 2, pk1 = pk0 + (left >> 2);
    for (int64_t j = pk0 + threadIdx.x; j < pk1; j += kAdamThreads) {
      const V4 p = ld_stream(reinterpret_cast<const V4*>(a.p[t]) + j), g = ld_stream(reinterpret_cast<const V4*>(a.g[t]) + j),
               m = ld_stream(reinterpret_cast<const V4*>(a.m[t]) + j), v = ld_stream(reinterpret_cast<const V4*>(a.v[t]) + j);
      V4 po, mo, vo;
#pragma unroll
      for (int e = 0; e < 4; ++e) adam_one<false>(p.v[e], g.v[e], m.v[e], v.v[e], a.h, d1, d2, po.v[e], mo.v[e], vo.v[e]);
      adam_multi_store(a, t, j, po, mo, vo);
    }
    for (int64_t k = (pk1 << 2) + threadIdx.x; k < a.n[t]; k += kAdamThreads) {
      float po, mo, vo;
      adam_one<false>(a.p[t][k], a.g[t][k], a.m[t][k], a.v[t][k], a.h, d1, d2, po, mo, vo);
      a.m[t][k] = mo;
      a.v[t][k] = vo;
      a.p[t][k] = po;
      if (a.lp_kind[t] == 1) store_lp_x1<1>(a.lp[t], k, po);
      if (a.lp_kind[t] == 2) store_lp_x1<2>(a.lp[t], k, po);
    }
  }
}

struct AdamMultiAttrs {
  AdamHyper h;
  uint32_t count;
  uint32_t lp_mask;
};
bool read_adam_multi(const void* attr, AdamMultiAttrs* out) {
  const AttrBlob& b = blob_of(attr);
  if (b.schema_id != schema::kAdam || !b.data || b.bytes < 32) return false;
  std::memcpy(&out->h, b.data, 24);
  std::memcpy(&out->count, static_cast<const uint8_t*>(b.data) + 24, 4);
  std::memcpy(&out->lp_mask, static_cast<const uint8_t*>(b.data) + 28, 4);
  return out->count >= 1 && out->count <= static_cast<uint32_t>(kMultiMax) && (out->lp_mask >> out->count) == 0;
}
bool adam_multi_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr, AdamMultiAttrs* at) {
  if (!in || !out || !read_adam_multi(attr, at)) return false;
  const int T = static_cast<int>(at->count);
  int lp_count = 0;
  for (int t = 0; t < T; ++t) lp_count += (at->lp_mask >> t) & 1u;
  if (ni != 4 * T + 1 || no != 3 * T + lp_count) return false;
  if (!i32_scalar(in[4 * T])) return false;
  int o = 0;
  for (int t = 0; t < T; ++t) {
    const TensorDesc* q = in + 4 * t;
    for (int i = 0; i < 4; ++i) {
      if (!f32_contig_rank1p(q[i]) || !same_shape(q[0], q[i]) || !aligned_to(q[i].data, 16)) return false;
      for (int j = 0; j < i; ++j)
        if (same_ptr(q[i], q[j])) return false;
    }
    // in place only: outputs are the parameter and its two moments themselves
    if (!same_ptr(out[o], q[0]) || !same_ptr(out[o + 1], q[2]) || !same_ptr(out[o + 2], q[3])) return false;
    for (int i = 0; i < 3; ++i)
      if (!f32_contig_rank1p(out[o + i]) || !same_shape(q[0], out[o + i])) return false;
    o += 3;
    if ((at->lp_mask >> t) & 1u) {
      const TensorDesc& lp = out[o++];
      if ((lp.dtype != DType::kBF16 && lp.dtype != DType::kF16) || !lp.contiguous || !same_shape(q[0], lp) || !aligned_to(lp.data, 8))
        return false;
    }
  }
  return true;
}
bool adam_multi_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  AdamMultiAttrs at;
  return adam_multi_check(in, ni, out, no, attr, &at);
}
Status adam_multi_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                         cudaStream_t stream) {
  AdamMultiAttrs at;
  if (!adam_multi_check(in, ni, out, no, attr, &at)) return Status::InvalidArgument;
  AdamMultiArgs a{};
  a.count = static_cast<int>(at.count);
  a.h = at.h;
  a.step = static_cast<const int32_t*>(in[4 * a.count].data);
  int o = 0;
  a.chunk_begin[0] = 0;
  for (int t = 0; t < a.count; ++t) {
    a.p[t] = static_cast<float*>(in[4 * t].data);
    a.g[t] = static_cast<const float*>(in[4 * t + 1].data);
    a.m[t] = static_cast<float*>(in[4 * t + 2].data);
    a.v[t] = static_cast<float*>(in[4 * t + 3].data);
    a.n[t] = numel_raw(in[4 * t]);
    a.chunk_begin[t + 1] = a.chunk_begin[t] + a.n[t] / kMultiChunk;
    o += 3;
    if ((at.lp_mask >> t) & 1u) {
      a.lp[t] = out[o].data;
      a.lp_kind[t] = out[o].dtype == DType::kBF16 ? 1 : 2;
      ++o;
    }
  }
  const int64_t work = a.chunk_begin[a.count] > a.count ? a.chunk_begin[a.count] : a.count;
  const int grid = streaming_grid(work, 1, kAdamBlocksPerSm);
  cudaGetLastError();
  adam_multi_kernel<<<grid, kAdamThreads, 0, stream>>>(a);
  return launch_status();
}

// ---------------------------------------------------------------- step_inc
// Contract (ops/step_inc/launcher.cu:92-144): int32, same shape, rank 0 allowed. The reference
// increments the OUTPUT buffer and never reads the input, so out-of-place use relies on the caller
// having copied the input first; that behaviour is kept.
__global__ void step_inc_kernel(int32_t* s, int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) s[i] += 1;
}
bool i32_ok(const TensorDesc& t) { return t.dtype == DType::kI32 && (t.rank() == 0 || t.contiguous); }
bool step_inc_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (!i32_ok(in[0]) || !i32_ok(out[0]) || !same_shape(in[0], out[0])) return false;
  int64_t n = 0;
  return positive_numel(in[0], 0, &n) && n >= 1;
}
bool step_inc_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return step_inc_check(in, ni, out, no);
}
Status step_inc_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t,
                       cudaStream_t stream) {
  if (!step_inc_check(in, ni, out, no)) return Status::InvalidArgument;
  int64_t n = 0;
  positive_numel(in[0], 0, &n);
  cudaGetLastError();
  step_inc_kernel<<<streaming_grid(n, 256, 4), 256, 0, stream>>>(static_cast<int32_t*>(out[0].data), n);
  return launch_status();
}

// ---------------------------------------------------------------- bias_corr
// step (i32 scalar) -> bc1_inv = 1/(1-beta1^t), bc2_inv = 1/(1-beta2^t), t = max(step,1), denominators
// clamped away from zero at 1e-20 (ops/biascorr/launcher.cu:82-101). Schema 'BCOR' is mandatory.
__global__ void bias_corr_kernel(const int32_t* step, float beta1, float beta2, float* o1, float* o2) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  int t = step[0];
  if (t < 1) t = 1;
  float d1 = 1.0f - powf(beta1, static_cast<float>(t));
  float d2 = 1.0f - powf(beta2, static_cast<float>(t));
  if (fabsf(d1) < 1e-20f) d1 = 1e-20f;
  if (fabsf(d2) < 1e-20f) d2 = 1e-20f;
  o1[0] = 1.0f / d1;
  o2[0] = 1.0f / d2;
}
bool scalar_like(const TensorDesc& d, DType dt) {
  return d.dtype == dt && d.contiguous && (d.rank() == 0 || (d.rank() == 1 && d.shape[0] == 1));
}
bool bias_corr_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr, float* betas) {
  if (!in || !out || ni != 1 || no != 2) return false;
  if (!scalar_like(in[0], DType::kI32) || !scalar_like(out[0], DType::kF32) || !scalar_like(out[1], DType::kF32))
    return false;
  float b[2];
  if (!read_attr_payload(attr, schema::kBiasCorr, false, b, 8)) return false;
  if (b[0] != b[0] || b[1] != b[1]) return false;  // NaN betas are rejected
  if (betas) {
    betas[0] = b[0];
    betas[1] = b[1];
  }
  return true;
}
bool bias_corr_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  return bias_corr_check(in, ni, out, no, attr, nullptr);
}
Status bias_corr_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                        cudaStream_t stream) {
  float b[2];
  if (!bias_corr_check(in, ni, out, no, attr, b)) return Status::InvalidArgument;
  cudaGetLastError();
  bias_corr_kernel<<<1, 32, 0, stream>>>(static_cast<const int32_t*>(in[0].data), b[0], b[1],
                                         static_cast<float*>(out[0].data), static_cast<float*>(out[1].data));
  return launch_status();
}

// ---------------------------------------------------------------- sgd_step
// O = P - lr*G, in place allowed, O must not alias G; lr from 'SGDS' <f>, default 1e-3
// (ops/sgd_step/launcher.cu:32-45,163-221). The update is computed in fp32 and rounded once.
template <typename T>
__global__ void __launch_bounds__(256) sgd_kernel(const T* p, const T* g, T* o, int64_t n, int64_t nvec, float lr) {
  using PK = Pack16<T>;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (int64_t i = tid; i < nvec; i += stride) {
    const PK a = ld_stream(reinterpret_cast<const PK*>(p) + i);
    const PK b = ld_stream(reinterpret_cast<const PK*>(g) + i);
    PK r;
#pragma unroll
    for (int e = 0; e < PK::kN; ++e) r.v[e] = Cvt<T>::from_f(Cvt<T>::to_f(a.v[e]) - lr * Cvt<T>::to_f(b.v[e]));
    st_stream(reinterpret_cast<PK*>(o) + i, r);
  }
  for (int64_t k = nvec * PK::kN + tid; k < n; k += stride)
    o[k] = Cvt<T>::from_f(Cvt<T>::to_f(p[k]) - lr * Cvt<T>::to_f(g[k]));
}
template <DType kDt>
bool sgd_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 2 || no != 1) return false;
  const TensorDesc* ts[] = {&in[0], &in[1], &out[0]};
  for (const TensorDesc* t : ts)
    if (t->dtype != kDt || !t->contiguous || t->rank() < 1) return false;
  if (!same_shape(in[0], in[1]) || !same_shape(in[0], out[0])) return false;
  int64_t n = 0;
  return positive_numel(in[0], 1, &n);
}
template <DType kDt>
bool sgd_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return sgd_check<kDt>(in, ni, out, no);
}
template <DType kDt, typename T>
Status sgd_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                  cudaStream_t stream) {
  if (!sgd_check<kDt>(in, ni, out, no)) return Status::InvalidArgument;
  if (out[0].data == in[1].data) return Status::InvalidArgument;
  float lr = 1e-3f;
  read_attr_payload(attr, schema::kSgd, false, &lr, 4);
  int64_t n = 0;
  positive_numel(in[0], 1, &n);
  const bool vec = aligned_to(in[0].data, 16) && aligned_to(in[1].data, 16) && aligned_to(out[0].data, 16);
  const int64_t nvec = vec ? n / Pack16<T>::kN : 0;
  cudaGetLastError();
  sgd_kernel<T><<<streaming_grid(vec ? nvec + 1 : n, 256, kStreamBlocksPerSm), 256, 0, stream>>>(
      static_cast<const T*>(in[0].data), static_cast<const T*>(in[1].data), static_cast<T*>(out[0].data), n, nvec, lr);
  return launch_status();
}

KernelVariant make(const char* name, uint32_t schema_gate,
                   Status (*launch)(const TensorDesc*, int, TensorDesc*, int, const void*, void*, size_t, cudaStream_t),
                   bool (*supported)(const TensorDesc*, int, const TensorDesc*, int, const void*)) {
  KernelVariant v{};
  v.name = name;
  v.flags = kKV_CaptureSafe;
  v.expected_attr_schema_id = schema_gate;
  v.launch = launch;
  v.supported = supported;
  v.query_workspace = no_workspace;
  return v;
}

}  // namespace

// Reads (optionally clears) the status word of the bulk-copy Adam kernel's bounded waits. Synchronises the device.
int adam_pipeline_status(bool) { return 0; }  // the Adam kernels have no device-side waits (they had, with a bulk-copy ring)

KernelVariant make_adam_step_f32_variant() { return make("adam_step_f32_sm100", schema::kAdam, adam_v0_launch, adam_v0_supported); }
KernelVariant make_adam_step_f32_fused_variant() { return make("adam_step_f32_fused_sm100", schema::kAdam, adam_v1_launch, adam_v1_supported); }
KernelVariant make_adam_step_f32_multi_variant() { return make("adam_step_f32_multi_sm100", schema::kAdam, adam_multi_launch, adam_multi_supported); }
KernelVariant make_step_inc_variant() { return make("step_inc_i32_sm100", 0, step_inc_launch, step_inc_supported); }
KernelVariant make_biascorr_variant() { return make("bias_corr_f32_sm100", schema::kBiasCorr, bias_corr_launch, bias_corr_supported); }
KernelVariant make_sgd_step_f32_variant() { return make("sgd_step_f32_sm100", 0, sgd_launch<DType::kF32, float>, sgd_supported<DType::kF32>); }
KernelVariant make_sgd_step_f16_variant() { return make("sgd_step_f16_sm100", 0, sgd_launch<DType::kF16, __half>, sgd_supported<DType::kF16>); }
KernelVariant make_sgd_step_bf16_variant() { return make("sgd_step_bf16_sm100", 0, sgd_launch<DType::kBF16, __nv_bfloat16>, sgd_supported<DType::kBF16>); }

}  // namespace aicf::cuda
