#pragma once
// Adam element maths and hyper-parameter payload shared by the single-device optimizer kernels and the
// data-parallel fused exchange+update kernel.
#include "common.cuh"

namespace aicf::cuda {

struct AdamHyper {
  float lr, beta1, beta2, eps;
  float weight_decay;  // 0 = none
  uint32_t decoupled;  // 0: L2 term folded into the gradient, 1: AdamW-style decay of the parameter
};

// 'ADAM' payload: <ffff> lr,beta1,beta2,eps, optionally followed by <fI> weight_decay, mode.
// Missing / foreign / short payloads fall back to the defaults the reference uses
// (ops/adam_step/launcher.cu:47-60).
inline AdamHyper read_adam(const void* attr) {
  AdamHyper h{1e-3f, 0.9f, 0.999f, 1e-8f, 0.0f, 0u};
  const AttrBlob& b = blob_of(attr);
  if (b.schema_id != schema::kAdam || !b.data || b.bytes < 16) return h;
  std::memcpy(&h, b.data, 16);
  if (b.bytes >= 24) {
    std::memcpy(&h.weight_decay, static_cast<const uint8_t*>(b.data) + 16, 4);
    std::memcpy(&h.decoupled, static_cast<const uint8_t*>(b.data) + 20, 4);
  }
  return h;
}

#ifdef __CUDACC__
template <bool kDivisorScalars>
__device__ __forceinline__ void adam_one(float p, float g, float m, float v, const AdamHyper& h, float d1,
                                         float d2, float& p_new, float& m_new, float& v_new) {
  if (!kDivisorScalars && h.weight_decay != 0.0f && h.decoupled == 0u) g = fmaf(h.weight_decay, p, g);
  m_new = h.beta1 * m + (1.0f - h.beta1) * g;
  v_new = h.beta2 * v + (1.0f - h.beta2) * (g * g);
  const float m_hat = m_new / d1;
  const float v_hat = v_new / d2;
  const float denom = sqrtf(v_hat) + h.eps;
  float base = p;
  if (!kDivisorScalars && h.weight_decay != 0.0f && h.decoupled != 0u) base = p - h.lr * h.weight_decay * p;
  p_new = base - h.lr * (m_hat / denom);
}

// kLp: 0 = no copy, 1 = bf16, 2 = f16
template <int kLp>
__device__ __forceinline__ void store_lp_x4(void* dst, int64_t packet, const Pack16<float>& f) {
  uint2 w;
  if (kLp == 1) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(f.v[0], f.v[1]);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(f.v[2], f.v[3]);
    w.x = *reinterpret_cast<const uint32_t*>(&lo);
    w.y = *reinterpret_cast<const uint32_t*>(&hi);
  } else {
    const __half2 lo = __floats2half2_rn(f.v[0], f.v[1]);
    const __half2 hi = __floats2half2_rn(f.v[2], f.v[3]);
    w.x = *reinterpret_cast<const uint32_t*>(&lo);
    w.y = *reinterpret_cast<const uint32_t*>(&hi);
  }
  reinterpret_cast<uint2*>(dst)[packet] = w;
}
template <int kLp>
__device__ __forceinline__ void store_lp_x1(void* dst, int64_t k, float v) {
  if (kLp == 1) static_cast<__nv_bfloat16*>(dst)[k] = __float2bfloat16_rn(v);
  if (kLp == 2) static_cast<__half*>(dst)[k] = __float2half_rn(v);
}

#endif  // __CUDACC__

}  // namespace aicf::cuda
