#pragma once
// Opaque per-op attribute payload: a schema tag plus little-endian POD bytes.
// Layout (16 bytes) matches the reference's attr_blob.hpp:13-17.
//   schema_id == 0  -> "unspecified", the op applies its defaults
//   bytes == 0 / data == nullptr are legal
#include <cstddef>
#include <cstdint>

namespace aicf::cuda {

struct AttrBlob {
  uint32_t schema_id = 0;
  uint32_t bytes = 0;
  const void* data = nullptr;
};

// Schema tags. The contract is the 32-bit value, not a spelling: the reference
// mixes big- and little-endian fourcc spellings, so the constants are kept verbatim
// (ops/gemm/launcher.cu:40, gemm_epilogue/launcher.cu:49, reduce_sum/launcher.cu:77,
// adam_step/launcher.cu:33, biascorr/launcher.cu:31, sgd_step/launcher.cu:32,
// bias_add/launcher.cu:96, mse_grad/launcher.cu:36).
namespace schema {
constexpr uint32_t kGemm = 0x47454D4Du;          // <ii>  transA, transB
constexpr uint32_t kGemmEpilogue = 0x4750454Cu;  // <iii> transA, transB, relu
constexpr uint32_t kReduceSum = 0x5253554Du;     // <q>   axis
constexpr uint32_t kAdam = 0x4D414441u;          // <ffff> lr,b1,b2,eps [+ <fI> weight_decay, mode]
constexpr uint32_t kBiasCorr = 0x524F4342u;      // <ff>  beta1, beta2
constexpr uint32_t kSgd = 0x53444753u;           // <f>   lr
constexpr uint32_t kBiasAdd = 0x44444142u;       // <q>   axis
constexpr uint32_t kMseGrad = 0x4745534Du;       // <f>   scale
constexpr uint32_t kLayerNorm = 0x50454E4Cu;
constexpr uint32_t kBatchNorm = 0x50454E42u;
// additions
constexpr uint32_t kSoftmaxCE = 0x45434D53u;     // 'SMCE' LE: <f> scale
constexpr uint32_t kAllReduce = 0x44455241u;     // 'ARED' LE: <i> bucket id
}  // namespace schema

}  // namespace aicf::cuda
