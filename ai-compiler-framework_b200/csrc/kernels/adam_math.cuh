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
// 1 / (1 - beta^t), t >= 1, in fp32 without the cancellation of 1 - powf(beta, t): beta^t - 1 = expm1(t * log1p(beta - 1)),
// where beta - 1 is exact (Sterbenz) and log1pf / expm1f are accurate to an ulp for small arguments. Relative error
// of the result about 2e-7 for every t (checked against double precision on the host for beta = 0.9 and 0.999,
// t = 1 .. 10^6); a thread computes both in ~60 fp32 instructions, where a double-precision pow() per thread costs
// thousands of cycles on a part with few fp64 units.
__device__ __forceinline__ void adam_inverse_corrections(const AdamHyper& h, int step, float& inv_d1, float& inv_d2) {
  const float t = static_cast<float>(step < 1 ? 1 : step);
  inv_d1 = 1.0f / -expm1f(t * log1pf(h.beta1 - 1.0f));
  inv_d2 = 1.0f / -expm1f(t * log1pf(h.beta2 - 1.0f));
}
__device__ __forceinline__ float sqrt_approx(float x) {  // max relative error 2^-23, sqrt(0) = 0
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float div_approx(float a, float b) {  // at most 2 ulp for 2^-126 <= |b| <= 2^126
  float r;
  asm("div.approx.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// One element. kDivisorScalars = true is the reference's contract (adam_step_f32_v0): c1, c2 are DIVISORS read from
// device scalars and every operation is the IEEE one the reference kernel uses (ops/adam_step/launcher.cu:269-291).
// kDivisorScalars = false is the fused contract: c1 = 1/(1-beta1^t), c2 = 1/(1-beta2^t) are MULTIPLIERS from
// adam_inverse_corrections, and the square root and the one remaining division are the hardware's single-instruction
// approximations (a few ulp together, against a tolerance of 1e-5): about 15 instructions per element instead of 40,
// which is what keeps the kernel bound by HBM and not by instruction issue when the SM clock drops under a power cap.
template <bool kDivisorScalars>
__device__ __forceinline__ void adam_one(float p, float g, float m, float v, const AdamHyper& h, float c1,
                                         float c2, float& p_new, float& m_new, float& v_new) {
  if (kDivisorScalars) {
    m_new = h.beta1 * m + (1.0f - h.beta1) * g;
    v_new = h.beta2 * v + (1.0f - h.beta2) * (g * g);
    const float m_hat = m_new / c1;
    const float v_hat = v_new / c2;
    p_new = p - h.lr * (m_hat / (sqrtf(v_hat) + h.eps));
    return;
  }
  if (h.weight_decay != 0.0f && h.decoupled == 0u) g = fmaf(h.weight_decay, p, g);
  m_new = h.beta1 * m + (1.0f - h.beta1) * g;
  v_new = h.beta2 * v + (1.0f - h.beta2) * (g * g);
  const float denom = sqrt_approx(v_new * c2) + h.eps;
  float base = p;
  if (h.weight_decay != 0.0f && h.decoupled != 0u) base = p - h.lr * h.weight_decay * p;
  p_new = base - h.lr * div_approx(m_new * c1, denom);
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
