#pragma once
// Argument checking and views shared by the two GEMM implementations (tcgen05 and SIMT).
#include "common.cuh"

namespace aicf::cuda {

// Logical 2-D operand after applying the transpose flag: element (r,c) lives at data[r*rs + c*cs].
struct MatView {
  const void* data = nullptr;
  int64_t rows = 0, cols = 0, rs = 0, cs = 0;
  DType dtype = DType::kUnknown;
};
inline MatView view_of(const TensorDesc& t, bool trans) {
  MatView v;
  v.data = t.data;
  v.dtype = t.dtype;
  v.rows = trans ? t.shape[1] : t.shape[0];
  v.cols = trans ? t.shape[0] : t.shape[1];
  v.rs = trans ? t.stride[1] : t.stride[0];
  v.cs = trans ? t.stride[0] : t.stride[1];
  return v;
}

struct GemmProblem {
  MatView A, B, C;     // A [M,K], B [K,N], C [M,N]
  const void* bias = nullptr;  // length N or null
  int64_t bias_stride = 1;
  DType bias_dtype = DType::kUnknown;
  bool relu = false;
  // optional ReLU-backward mask: C[m,n] is zeroed where mask[m,n] <= 0 (same dtype as C, unit column stride)
  const void* mask = nullptr;
  int64_t mask_ld = 0;
  int64_t M = 0, N = 0, K = 0;
};

// 'GEMM' <ii> transA,transB; schema 0 or a foreign schema or a short payload -> no transposes
// (ops/gemm/launcher.cu:48-70).
inline void read_gemm_attr(const void* attr, bool* ta, bool* tb) {
  int32_t p[2] = {0, 0};
  *ta = *tb = false;
  if (read_attr_payload(attr, schema::kGemm, true, p, 8)) {
    *ta = p[0] != 0;
    *tb = p[1] != 0;
  }
}
// 'GPEL' <iii> transA,transB,relu; anything else -> no transposes, relu ON
// (ops/gemm_epilogue/launcher.cu:57-80). A payload sent under another schema id is ignored, which is
// what the reference does with the executor's 'GEPI' tag.
inline void read_gemm_epilogue_attr(const void* attr, bool* ta, bool* tb, bool* relu) {
  int32_t p[3] = {0, 0, 1};
  *ta = *tb = false;
  *relu = true;
  if (read_attr_payload(attr, schema::kGemmEpilogue, true, p, 12)) {
    *ta = p[0] != 0;
    *tb = p[1] != 0;
    *relu = p[2] != 0;
  }
}

// Shape/stride validation common to gemm and gemm_epilogue (ops/gemm/launcher.cu:116-148,
// ops/gemm_epilogue/launcher.cu:146-193). dtype rules are applied by the caller.
inline bool build_problem(const TensorDesc* in, int ni, const TensorDesc* out, int no, bool with_bias, bool ta, bool tb,
                          bool relu, GemmProblem* p) {
  if (!in || !out || no != 1 || ni != (with_bias ? 3 : 2)) return false;
  const TensorDesc &A0 = in[0], &B0 = in[1], &C0 = out[0];
  if (A0.rank() != 2 || B0.rank() != 2 || C0.rank() != 2) return false;
  for (const TensorDesc* t : {&A0, &B0, &C0})
    if (t->stride[0] <= 0 || t->stride[1] <= 0) return false;
  p->A = view_of(A0, ta);
  p->B = view_of(B0, tb);
  p->C = view_of(C0, false);
  p->M = p->A.rows;
  p->K = p->A.cols;
  p->N = p->B.cols;
  if (p->M <= 0 || p->N <= 0 || p->K <= 0) return false;
  if (p->B.rows != p->K || p->C.rows != p->M || p->C.cols != p->N) return false;
  p->relu = relu;
  if (with_bias) {
    const TensorDesc& b = in[2];
    if (b.rank() != 1 || b.stride[0] <= 0 || b.shape[0] != p->N) return false;
    p->bias = b.data;
    p->bias_stride = b.stride[0];
    p->bias_dtype = b.dtype;
  }
  return true;
}

// Implemented in gemm_simt.cu: tiled FFMA kernel for any strides and any of f32/f16/bf16 operands.
Status gemm_simt_run(const GemmProblem& p, cudaStream_t stream);
// Implemented in gemm_tcgen05.cu: returns NotImplemented when the problem does not meet the TMA
// alignment rules, so the caller can fall through to the SIMT kernel.
// `ws` (may be null) is scratch of at least gemm_tcgen05_workspace(p) bytes: with it, a product that has few tiles
// and a long K is split over K; without it the same product runs unsplit.
Status gemm_tcgen05_run(const GemmProblem& p, void* ws, size_t ws_bytes, cudaStream_t stream);
size_t gemm_tcgen05_workspace(const GemmProblem& p);
bool gemm_tcgen05_eligible(const GemmProblem& p);
// Implemented in gemm_tcgen05.cu: fp32 operands on the tensor cores as three TF32 products per k step (hi/lo split
// of both operands, staged in `ws`). Not bit-identical to an fp32 FMA chain; error is of the order of fp32 rounding.
bool gemm_tf32x3_eligible(const GemmProblem& p);
size_t gemm_tf32x3_workspace(const GemmProblem& p);
Status gemm_tf32x3_run(const GemmProblem& p, void* ws, size_t ws_bytes, cudaStream_t stream);

}  // namespace aicf::cuda
