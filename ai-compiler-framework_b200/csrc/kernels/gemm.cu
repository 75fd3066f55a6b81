// Kernel variants of OpKind::Gemm, OpKind::GemmEpilogue and OpKind::GemmReluBwd.
//
// Each variant validates its contract and then routes to one of two sm_100a kernels:
//   gemm_tcgen05_run  16-bit operands whose rows are 16-byte aligned (TMA + tcgen05/TMEM)
//   gemm_simt_run     fp32 operands (exact fp32), or shapes the TMA path cannot express
//   gemm_tf32x3_run   fp32 operands on the tensor cores (three TF32 products per k step), only under its own ids
// The reference ids keep the reference's dtype contracts
// (ops/gemm/launcher.cu:272-287,330-361; ops/gemm_epilogue/launcher.cu:333-349,399-431).
#include "gemm_common.cuh"

namespace aicf::cuda {

namespace {

enum class BiasRule { None, SameAsInput, F32OrInput, ReluBwdMask };  // the last: third input is the activation Y

struct GemmContract {
  DType in, out;
  BiasRule bias;
  bool c_rowmajor_contig;  // the reference's tensor-core ids insist on a packed row-major C
};

bool is_packed_rowmajor(const TensorDesc& t) { return t.rank() == 2 && t.stride[1] == 1 && t.stride[0] == t.shape[1]; }

bool check(const GemmContract& c, const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr,
           GemmProblem* prob) {
  const bool with_mask = c.bias == BiasRule::ReluBwdMask;
  const bool with_bias = c.bias != BiasRule::None && !with_mask;
  bool ta, tb, relu = false;
  if (with_mask) {
    // inputs [dY, W, Y] -> dX: shape rules of gemm on the first two, Y must look exactly like the output
    if (!in || ni != 3) return false;
    read_gemm_attr(attr, &ta, &tb);
    GemmProblem pm;
    if (!build_problem(in, 2, out, no, false, ta, tb, false, &pm)) return false;
    if (in[0].dtype != c.in || in[1].dtype != c.in || out[0].dtype != c.out) return false;
    const TensorDesc& Y = in[2];
    if (Y.dtype != c.out || Y.rank() != 2 || Y.shape[0] != pm.M || Y.shape[1] != pm.N || Y.stride[1] != 1 || Y.stride[0] < pm.N)
      return false;
    pm.mask = Y.data;
    pm.mask_ld = Y.stride[0];
    if (prob) *prob = pm;
    return true;
  }
  if (with_bias) {
    read_gemm_epilogue_attr(attr, &ta, &tb, &relu);
  } else {
    read_gemm_attr(attr, &ta, &tb);
  }
  GemmProblem p;
  if (!build_problem(in, ni, out, no, with_bias, ta, tb, relu, &p)) return false;
  if (in[0].dtype != c.in || in[1].dtype != c.in || out[0].dtype != c.out) return false;
  if (with_bias) {
    const DType bd = in[2].dtype;
    if (c.bias == BiasRule::SameAsInput && bd != c.in) return false;
    if (c.bias == BiasRule::F32OrInput && bd != DType::kF32 && bd != c.in) return false;
  }
  if (c.c_rowmajor_contig && !is_packed_rowmajor(out[0])) return false;
  if (prob) *prob = p;
  return true;
}

Status run(const GemmProblem& p, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (gemm_tcgen05_eligible(p)) return gemm_tcgen05_run(p, ws, ws_bytes, stream);
  return gemm_simt_run(p, stream);
}

size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }

template <int kId> struct Contracts;
#define AICF_GEMM_CONTRACT(ID, IN, OUT, BIAS, PACKED)                                                              \
  template <> struct Contracts<ID> {                                                                              \
    static constexpr GemmContract value{IN, OUT, BIAS, PACKED};                                                   \
  };
AICF_GEMM_CONTRACT(0, DType::kF32, DType::kF32, BiasRule::None, false)
AICF_GEMM_CONTRACT(1, DType::kF16, DType::kF16, BiasRule::None, true)
AICF_GEMM_CONTRACT(2, DType::kBF16, DType::kBF16, BiasRule::None, false)
AICF_GEMM_CONTRACT(3, DType::kBF16, DType::kF32, BiasRule::None, false)
AICF_GEMM_CONTRACT(4, DType::kF16, DType::kF32, BiasRule::None, false)
AICF_GEMM_CONTRACT(5, DType::kF16, DType::kF16, BiasRule::None, false)
AICF_GEMM_CONTRACT(10, DType::kF32, DType::kF32, BiasRule::SameAsInput, false)
AICF_GEMM_CONTRACT(11, DType::kF16, DType::kF16, BiasRule::SameAsInput, true)
AICF_GEMM_CONTRACT(12, DType::kBF16, DType::kBF16, BiasRule::F32OrInput, false)
AICF_GEMM_CONTRACT(13, DType::kBF16, DType::kF32, BiasRule::F32OrInput, false)
AICF_GEMM_CONTRACT(14, DType::kF16, DType::kF16, BiasRule::F32OrInput, false)
AICF_GEMM_CONTRACT(20, DType::kBF16, DType::kBF16, BiasRule::ReluBwdMask, false)
AICF_GEMM_CONTRACT(21, DType::kF16, DType::kF16, BiasRule::ReluBwdMask, false)
AICF_GEMM_CONTRACT(22, DType::kF32, DType::kF32, BiasRule::ReluBwdMask, false)

template <int kId>
bool supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  return check(Contracts<kId>::value, in, ni, out, no, attr, nullptr);
}
template <int kId>
Status launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void* ws, size_t ws_bytes,
              cudaStream_t stream) {
  GemmProblem p;
  if (!check(Contracts<kId>::value, in, ni, out, no, attr, &p)) return Status::InvalidArgument;
  return run(p, ws, ws_bytes, stream);
}
// Workspace of the tensor-core path (split-K parts). The output is not known here; its dtype and layout follow from
// the contract (dtype kId's out, packed rows), which is all the eligibility test and the size need.
template <int kId>
size_t gemm_workspace(const TensorDesc* in, int ni, const void* attr) {
  constexpr GemmContract c = Contracts<kId>::value;
  if (c.in == DType::kF32 || !in || ni < 2 || in[0].rank() != 2 || in[1].rank() != 2) return 0;
  bool ta, tb, relu;
  if (c.bias == BiasRule::None || c.bias == BiasRule::ReluBwdMask) read_gemm_attr(attr, &ta, &tb);
  else read_gemm_epilogue_attr(attr, &ta, &tb, &relu);
  GemmProblem p;
  p.A = view_of(in[0], ta);
  p.B = view_of(in[1], tb);
  p.M = p.A.rows;
  p.K = p.A.cols;
  p.N = p.B.cols;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.B.rows != p.K) return 0;
  p.C.dtype = c.out;
  p.C.rows = p.M;
  p.C.cols = p.N;
  p.C.rs = p.N;
  p.C.cs = 1;
  return gemm_tcgen05_workspace(p);
}
// fp32 on the tensor cores: opt-in ids, never chosen over the exact kernel by priority dispatch (lower priority).
template <int kId>
size_t tf32x3_workspace(const TensorDesc* in, int ni, const void* attr) {
  if (!in || ni < 2 || in[0].rank() != 2 || in[1].rank() != 2) return 0;
  bool ta, tb, relu;
  if (Contracts<kId>::value.bias == BiasRule::None || Contracts<kId>::value.bias == BiasRule::ReluBwdMask)
    read_gemm_attr(attr, &ta, &tb);
  else
    read_gemm_epilogue_attr(attr, &ta, &tb, &relu);
  GemmProblem p;
  p.A = view_of(in[0], ta);
  p.B = view_of(in[1], tb);
  p.M = p.A.rows;
  p.K = p.A.cols;
  p.N = p.B.cols;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return 0;
  return gemm_tf32x3_workspace(p);
}
template <int kId>
bool tf32x3_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  GemmProblem p;
  return check(Contracts<kId>::value, in, ni, out, no, attr, &p) && gemm_tf32x3_eligible(p);
}
template <int kId>
Status tf32x3_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void* ws, size_t ws_bytes,
                     cudaStream_t stream) {
  GemmProblem p;
  if (!check(Contracts<kId>::value, in, ni, out, no, attr, &p) || !gemm_tf32x3_eligible(p)) return Status::InvalidArgument;
  return gemm_tf32x3_run(p, ws, ws_bytes, stream);
}
template <int kId>
KernelVariant tf32x3_variant(const char* name) {
  KernelVariant v{};
  v.name = name;
  v.flags = kKV_CaptureSafe;
  v.expected_attr_schema_id = 0;
  v.launch = tf32x3_launch<kId>;
  v.supported = tf32x3_supported<kId>;
  v.query_workspace = tf32x3_workspace<kId>;
  return v;
}

template <int kId>
KernelVariant variant(const char* name) {
  KernelVariant v{};
  v.name = name;
  v.flags = kKV_CaptureSafe;
  v.expected_attr_schema_id = 0;  // schema 0 and the op's own schema are both parsed
  v.launch = launch<kId>;
  v.supported = supported<kId>;
  v.query_workspace = gemm_workspace<kId>;
  return v;
}

}  // namespace

KernelVariant make_gemm_f32_naive_variant() { return variant<0>("gemm_f32_simt_sm100"); }
KernelVariant make_gemm_f16_tc_wmma_out_f16_variant() { return variant<1>("gemm_f16_tcgen05_packed_c"); }
KernelVariant make_gemm_bf16_tcgen05_out_bf16_variant() { return variant<2>("gemm_bf16_tcgen05_out_bf16"); }
KernelVariant make_gemm_bf16_tcgen05_out_f32_variant() { return variant<3>("gemm_bf16_tcgen05_out_f32"); }
KernelVariant make_gemm_f16_tcgen05_out_f32_variant() { return variant<4>("gemm_f16_tcgen05_out_f32"); }
KernelVariant make_gemm_f16_tcgen05_out_f16_variant() { return variant<5>("gemm_f16_tcgen05_out_f16"); }
KernelVariant make_gemm_bias_relu_f32_naive_variant() { return variant<10>("gemm_bias_relu_f32_simt_sm100"); }
KernelVariant make_gemm_bias_relu_f16_tc_wmma_out_f16_variant() { return variant<11>("gemm_bias_relu_f16_tcgen05_packed_c"); }
KernelVariant make_gemm_bias_relu_bf16_tcgen05_out_bf16_variant() { return variant<12>("gemm_bias_relu_bf16_tcgen05_out_bf16"); }
KernelVariant make_gemm_bias_relu_bf16_tcgen05_out_f32_variant() { return variant<13>("gemm_bias_relu_bf16_tcgen05_out_f32"); }
KernelVariant make_gemm_bias_relu_f16_tcgen05_out_f16_variant() { return variant<14>("gemm_bias_relu_f16_tcgen05_out_f16"); }

KernelVariant make_gemm_f32_3xtf32_variant() { return tf32x3_variant<0>("gemm_f32_3xtf32_tcgen05"); }
KernelVariant make_gemm_bias_relu_f32_3xtf32_variant() { return tf32x3_variant<10>("gemm_bias_relu_f32_3xtf32_tcgen05"); }
KernelVariant make_gemm_relu_bwd_f32_3xtf32_variant() { return tf32x3_variant<22>("gemm_relu_bwd_f32_3xtf32_tcgen05"); }

KernelVariant make_gemm_relu_bwd_bf16_variant() { return variant<20>("gemm_relu_bwd_bf16_tcgen05"); }
KernelVariant make_gemm_relu_bwd_f16_variant() { return variant<21>("gemm_relu_bwd_f16_tcgen05"); }
KernelVariant make_gemm_relu_bwd_f32_variant() { return variant<22>("gemm_relu_bwd_f32_simt_sm100"); }

}  // namespace aicf::cuda
