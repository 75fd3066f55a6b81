// Elementwise ops of the MLP train step: relu, relu_bwd, bias_add, add, copy, mse_grad, cast and
// grad_zero. All are one-pass HBM-bound kernels built from one template: 16-byte packets with
// evict-first hints, 64-bit grid-stride indexing (no element-count ceiling; the reference's relu
// rejects numel > INT_MAX and its relu_bwd silently skips elements past 65535*256), scalar path for
// the ragged tail or unaligned views. Grids are as large as the array needs at two packets per thread, up to
// kStreamBlocksPerSm blocks per SM.
#include "common.cuh"

namespace aicf::cuda {

namespace {

size_t no_workspace(const TensorDesc*, int, const void*) { return 0; }

// ---- generic 1/2-input elementwise kernel ------------------------------------------------------
template <typename T, int kInputs, typename F>
__global__ void __launch_bounds__(256) eltwise_kernel(const T* a, const T* b, T* o, int64_t n, int64_t nvec, F f) {
  using PK = Pack16<T>;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t i = tid;
  for (; i + stride < nvec; i += 2 * stride) {  // two packets in flight per input
    PK x0 = ld_stream(reinterpret_cast<const PK*>(a) + i), x1 = ld_stream(reinterpret_cast<const PK*>(a) + i + stride);
    PK y0 = x0, y1 = x1;
    if (kInputs == 2) {
      y0 = ld_stream(reinterpret_cast<const PK*>(b) + i);
      y1 = ld_stream(reinterpret_cast<const PK*>(b) + i + stride);
    }
    PK r0, r1;
#pragma unroll
    for (int e = 0; e < PK::kN; ++e) {
      r0.v[e] = Cvt<T>::from_f(f(Cvt<T>::to_f(x0.v[e]), Cvt<T>::to_f(y0.v[e])));
      r1.v[e] = Cvt<T>::from_f(f(Cvt<T>::to_f(x1.v[e]), Cvt<T>::to_f(y1.v[e])));
    }
    st_stream(reinterpret_cast<PK*>(o) + i, r0);
    st_stream(reinterpret_cast<PK*>(o) + i + stride, r1);
  }
  for (; i < nvec; i += stride) {
    const PK x = ld_stream(reinterpret_cast<const PK*>(a) + i);
    PK y = x;
    if (kInputs == 2) y = ld_stream(reinterpret_cast<const PK*>(b) + i);
    PK r;
#pragma unroll
    for (int e = 0; e < PK::kN; ++e) r.v[e] = Cvt<T>::from_f(f(Cvt<T>::to_f(x.v[e]), Cvt<T>::to_f(y.v[e])));
    st_stream(reinterpret_cast<PK*>(o) + i, r);
  }
  for (int64_t k = nvec * PK::kN + tid; k < n; k += stride) {
    const float x = Cvt<T>::to_f(a[k]);
    const float y = kInputs == 2 ? Cvt<T>::to_f(b[k]) : x;
    o[k] = Cvt<T>::from_f(f(x, y));
  }
}

template <typename T, int kInputs, typename F>
Status run_eltwise(const void* a, const void* b, void* o, int64_t n, F f, cudaStream_t stream) {
  if (n <= 0) return Status::Ok;
  const bool vec = aligned_to(a, 16) && aligned_to(o, 16) && (kInputs == 1 || aligned_to(b, 16));
  const int64_t nvec = vec ? n / Pack16<T>::kN : 0;
  const int grid = streaming_grid(vec ? nvec / 2 + 1 : n, 256, kStreamBlocksPerSm);
  cudaGetLastError();
  eltwise_kernel<T, kInputs, F><<<grid, 256, 0, stream>>>(static_cast<const T*>(a), static_cast<const T*>(b),
                                                         static_cast<T*>(o), n, nvec, f);
  return launch_status();
}

struct ReluF { __device__ float operator()(float x, float) const { return x > 0.0f ? x : 0.0f; } };
struct ReluBwdF { __device__ float operator()(float dout, float y) const { return y > 0.0f ? dout : 0.0f; } };
struct AddF { __device__ float operator()(float x, float y) const { return x + y; } };
struct CopyF { __device__ float operator()(float x, float) const { return x; } };
struct MseGradF {
  float scale;
  __device__ float operator()(float pred, float target) const { return (pred - target) * scale; }
};

template <DType kDt> struct CType;
template <> struct CType<DType::kF32> { using type = float; };
template <> struct CType<DType::kF16> { using type = __half; };
template <> struct CType<DType::kBF16> { using type = __nv_bfloat16; };

bool contig_by_strides(const TensorDesc& t) {
  const int r = t.rank();
  if (r <= 0) return false;
  int64_t expect = 1;
  for (int i = r - 1; i >= 0; --i) {
    if (t.stride[i] != expect) return false;
    expect *= t.shape[i];
  }
  return true;
}

// ---- relu: (X) -> (Y), same shape/dtype, contiguity judged from strides (ops/relu/launcher.cu:90-133)
template <DType kDt>
bool relu_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != kDt || out[0].dtype != kDt || !same_shape(in[0], out[0])) return false;
  if (!contig_by_strides(in[0]) || !contig_by_strides(out[0])) return false;
  int64_t n = 0;
  return positive_numel(out[0], 1, &n);
}
template <DType kDt>
bool relu_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return relu_check<kDt>(in, ni, out, no);
}
template <DType kDt>
Status relu_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!relu_check<kDt>(in, ni, out, no)) return Status::InvalidArgument;
  using T = typename CType<kDt>::type;
  return run_eltwise<T, 1>(in[0].data, nullptr, out[0].data, out[0].numel(), ReluF{}, s);
}

// ---- two-input family: relu_bwd (dOut, Y) -> dY; add (A,B) -> O; mse_grad (pred,target) -> grad
template <DType kDt>
bool binary_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, int min_rank) {
  if (!in || !out || ni != 2 || no != 1) return false;
  const TensorDesc* ts[] = {&in[0], &in[1], &out[0]};
  for (const TensorDesc* t : ts)
    if (t->dtype != kDt || !t->contiguous) return false;
  if (!same_shape(in[0], in[1]) || !same_shape(in[0], out[0])) return false;
  int64_t n = 0;
  return positive_numel(in[0], min_rank, &n);
}
template <DType kDt>
bool relu_bwd_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return binary_check<kDt>(in, ni, out, no, 1);
}
template <DType kDt>
Status relu_bwd_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!binary_check<kDt>(in, ni, out, no, 1)) return Status::InvalidArgument;
  using T = typename CType<kDt>::type;
  return run_eltwise<T, 2>(in[0].data, in[1].data, out[0].data, in[0].numel(), ReluBwdF{}, s);
}
template <DType kDt>
bool add_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return binary_check<kDt>(in, ni, out, no, 0);
}
template <DType kDt>
Status add_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!binary_check<kDt>(in, ni, out, no, 0)) return Status::InvalidArgument;
  using T = typename CType<kDt>::type;
  return run_eltwise<T, 2>(in[0].data, in[1].data, out[0].data, in[0].numel(), AddF{}, s);
}
// mse_grad: scale from 'MSEG' <f>, otherwise 2/numel (ops/mse_grad/launcher.cu:36-52,213-215)
template <DType kDt>
bool mse_grad_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return binary_check<kDt>(in, ni, out, no, 1);
}
template <DType kDt>
Status mse_grad_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                       cudaStream_t s) {
  if (!binary_check<kDt>(in, ni, out, no, 1)) return Status::InvalidArgument;
  using T = typename CType<kDt>::type;
  const int64_t n = in[0].numel();
  float scale = 0.0f;
  if (!read_attr_payload(attr, schema::kMseGrad, false, &scale, 4)) scale = 2.0f / static_cast<float>(n);
  return run_eltwise<T, 2>(in[0].data, in[1].data, out[0].data, n, MseGradF{scale}, s);
}

// ---- copy: (X) -> (Y) same dtype/shape, contiguous; empty tensors are a no-op (ops/copy/launcher.cu:66-110)
template <DType kDt>
bool copy_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != kDt || out[0].dtype != kDt) return false;
  return in[0].contiguous && out[0].contiguous && same_shape(in[0], out[0]);
}
template <DType kDt>
bool copy_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return copy_check<kDt>(in, ni, out, no);
}
int64_t numel_or_zero(const TensorDesc& t) {
  int64_t n = 0;
  return positive_numel(t, 1, &n) ? n : 0;
}
template <DType kDt>
Status copy_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!copy_check<kDt>(in, ni, out, no)) return Status::InvalidArgument;
  using T = typename CType<kDt>::type;
  if (in[0].data == out[0].data) return Status::Ok;
  return run_eltwise<T, 1>(in[0].data, nullptr, out[0].data, numel_or_zero(in[0]), CopyF{}, s);
}
// int32 copy (step counters) moves raw bits through the f32 path
bool copy_i32_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return copy_check<DType::kI32>(in, ni, out, no);
}
Status copy_i32_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!copy_check<DType::kI32>(in, ni, out, no)) return Status::InvalidArgument;
  const int64_t n = numel_or_zero(in[0]);
  if (n == 0 || in[0].data == out[0].data) return Status::Ok;
  return status_of(cudaMemcpyAsync(out[0].data, in[0].data, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, s));
}

// ---- grad_zero: memset node (ops/grad_zero/launcher.cu:60-119); bf16 and i32 added
bool grad_zero_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (in[0].dtype != out[0].dtype || !same_shape(in[0], out[0])) return false;
  if (!in[0].contiguous || !out[0].contiguous) return false;
  return dtype_size_bytes(in[0].dtype) != 0;
}
bool grad_zero_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return grad_zero_check(in, ni, out, no);
}
Status grad_zero_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!grad_zero_check(in, ni, out, no)) return Status::InvalidArgument;
  const int64_t n = numel_or_zero(out[0]);
  if (n == 0) return Status::Ok;
  cudaGetLastError();
  return status_of(cudaMemsetAsync(out[0].data, 0, static_cast<size_t>(n) * dtype_size_bytes(out[0].dtype), s));
}

// ---- bias_add: Out[..., c] = Y[..., c] + bias[c]; last axis only (ops/bias_add/launcher.cu:98-196)
// Packets never straddle a row when N is a multiple of the packet width, so the column of a packet
// is (packet_index % (N/kN)) * kN: one modulo per 16 bytes instead of one per element.
template <typename T>
__global__ void __launch_bounds__(256) bias_add_kernel(const T* y, const T* bias, T* o, int64_t total, int64_t N,
                                                      int vec_ok) {
  using PK = Pack16<T>;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec_ok) {
    const int64_t nvec = total / PK::kN, ncol_v = N / PK::kN;
    for (int64_t i = tid; i < nvec; i += stride) {
      const PK a = ld_stream(reinterpret_cast<const PK*>(y) + i);
      const PK b = *(reinterpret_cast<const PK*>(bias) + (i % ncol_v));
      PK r;
#pragma unroll
      for (int e = 0; e < PK::kN; ++e) r.v[e] = Cvt<T>::from_f(Cvt<T>::to_f(a.v[e]) + Cvt<T>::to_f(b.v[e]));
      st_stream(reinterpret_cast<PK*>(o) + i, r);
    }
  } else {
    for (int64_t k = tid; k < total; k += stride) o[k] = Cvt<T>::from_f(Cvt<T>::to_f(y[k]) + Cvt<T>::to_f(bias[k % N]));
  }
}
int64_t read_axis_bias_add(const void* attr) {
  int64_t axis = -1;
  read_attr_payload(attr, schema::kBiasAdd, true, &axis, 8);
  return axis;
}
template <DType kDt>
bool bias_add_check(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  if (!in || !out || ni != 2 || no != 1) return false;
  const TensorDesc &Y = in[0], &B = in[1], &O = out[0];
  if (Y.dtype != kDt || !Y.contiguous || Y.rank() < 2) return false;
  if (O.dtype != kDt || !O.contiguous || O.rank() < 2) return false;
  if (B.dtype != kDt || !B.contiguous || B.rank() != 1) return false;
  const int64_t axis = read_axis_bias_add(attr);
  if (axis != -1 && axis != Y.rank() - 1) return false;
  if (!same_shape(Y, O)) return false;
  int64_t M = 0, N = 0;
  return rows_cols_lastdim(Y, &M, &N) && B.shape[0] == N;
}
template <DType kDt>
bool bias_add_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void* attr) {
  return bias_add_check<kDt>(in, ni, out, no, attr);
}
template <DType kDt>
Status bias_add_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void* attr, void*, size_t,
                       cudaStream_t s) {
  if (!bias_add_check<kDt>(in, ni, out, no, attr)) return Status::InvalidArgument;
  using T = typename CType<kDt>::type;
  int64_t M = 0, N = 0;
  rows_cols_lastdim(in[0], &M, &N);
  const int64_t total = M * N;
  const int vec = (N % Pack16<T>::kN == 0) && aligned_to(in[0].data, 16) && aligned_to(in[1].data, 16) &&
                  aligned_to(out[0].data, 16);
  cudaGetLastError();
  bias_add_kernel<T><<<streaming_grid(vec ? total / Pack16<T>::kN : total, 256, kStreamBlocksPerSm), 256, 0, s>>>(
      static_cast<const T*>(in[0].data), static_cast<const T*>(in[1].data), static_cast<T*>(out[0].data), total, N, vec);
  return launch_status();
}

// ---- cast: (X) -> (Y), same shape, any pair of {f32,f16,bf16}; round-to-nearest-even
template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_kernel(const S* x, D* y, int64_t n, int vec_ok) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  constexpr int kW = 8;  // elements per trip on the vector path
  const int64_t nvec = vec_ok ? n / kW : 0;
  for (int64_t i = tid; i < nvec; i += stride) {
    S src[kW];
    D dst[kW];
    constexpr int kSrcPk = (kW * sizeof(S)) / 16, kDstPk = (kW * sizeof(D)) / 16;
#pragma unroll
    for (int q = 0; q < kSrcPk; ++q)
      reinterpret_cast<int4*>(src)[q] = __ldcs(reinterpret_cast<const int4*>(x) + i * kSrcPk + q);
#pragma unroll
    for (int e = 0; e < kW; ++e) dst[e] = Cvt<D>::from_f(Cvt<S>::to_f(src[e]));
#pragma unroll
    for (int q = 0; q < kDstPk; ++q) __stcs(reinterpret_cast<int4*>(y) + i * kDstPk + q, reinterpret_cast<int4*>(dst)[q]);
  }
  for (int64_t k = nvec * kW + tid; k < n; k += stride) y[k] = Cvt<D>::from_f(Cvt<S>::to_f(x[k]));
}
bool cast_check(const TensorDesc* in, int ni, const TensorDesc* out, int no) {
  if (!in || !out || ni != 1 || no != 1) return false;
  if (!dtype_is_float(in[0].dtype) || !dtype_is_float(out[0].dtype)) return false;
  if (!in[0].contiguous || !out[0].contiguous || !same_shape(in[0], out[0])) return false;
  int64_t n = 0;
  return positive_numel(in[0], 1, &n);
}
bool cast_supported(const TensorDesc* in, int ni, const TensorDesc* out, int no, const void*) {
  return cast_check(in, ni, out, no);
}
template <typename S, typename D>
Status cast_run(const TensorDesc& x, TensorDesc& y, cudaStream_t s) {
  const int64_t n = x.numel();
  const int vec = aligned_to(x.data, 16) && aligned_to(y.data, 16);
  cudaGetLastError();
  cast_kernel<S, D><<<streaming_grid(vec ? n / 8 + 1 : n, 256, kStreamBlocksPerSm), 256, 0, s>>>(static_cast<const S*>(x.data),
                                                                               static_cast<D*>(y.data), n, vec);
  return launch_status();
}
template <typename S>
Status cast_from(const TensorDesc& x, TensorDesc& y, cudaStream_t s) {
  switch (y.dtype) {
    case DType::kF32: return cast_run<S, float>(x, y, s);
    case DType::kF16: return cast_run<S, __half>(x, y, s);
    case DType::kBF16: return cast_run<S, __nv_bfloat16>(x, y, s);
    default: return Status::InvalidArgument;
  }
}
Status cast_launch(const TensorDesc* in, int ni, TensorDesc* out, int no, const void*, void*, size_t, cudaStream_t s) {
  if (!cast_check(in, ni, out, no)) return Status::InvalidArgument;
  switch (in[0].dtype) {
    case DType::kF32: return cast_from<float>(in[0], out[0], s);
    case DType::kF16: return cast_from<__half>(in[0], out[0], s);
    case DType::kBF16: return cast_from<__nv_bfloat16>(in[0], out[0], s);
    default: return Status::InvalidArgument;
  }
}

using LaunchFn = Status (*)(const TensorDesc*, int, TensorDesc*, int, const void*, void*, size_t, cudaStream_t);
using SupportedFn = bool (*)(const TensorDesc*, int, const TensorDesc*, int, const void*);
KernelVariant make(const char* name, LaunchFn l, SupportedFn s) {
  KernelVariant v{};
  v.name = name;
  v.flags = kKV_CaptureSafe;
  v.launch = l;
  v.supported = s;
  v.query_workspace = no_workspace;
  return v;
}

}  // namespace

#define AICF_ELTWISE_FACTORY(fn, nm, L, S) \
  KernelVariant fn() { return make(nm, L, S); }

AICF_ELTWISE_FACTORY(make_relu_f32_variant, "relu_f32_sm100", relu_launch<DType::kF32>, relu_supported<DType::kF32>)
AICF_ELTWISE_FACTORY(make_relu_f16_variant, "relu_f16_sm100", relu_launch<DType::kF16>, relu_supported<DType::kF16>)
AICF_ELTWISE_FACTORY(make_relu_bf16_variant, "relu_bf16_sm100", relu_launch<DType::kBF16>, relu_supported<DType::kBF16>)
AICF_ELTWISE_FACTORY(make_relu_bwd_f32_variant, "relu_bwd_f32_sm100", relu_bwd_launch<DType::kF32>, relu_bwd_supported<DType::kF32>)
AICF_ELTWISE_FACTORY(make_relu_bwd_f16_variant, "relu_bwd_f16_sm100", relu_bwd_launch<DType::kF16>, relu_bwd_supported<DType::kF16>)
AICF_ELTWISE_FACTORY(make_relu_bwd_bf16_variant, "relu_bwd_bf16_sm100", relu_bwd_launch<DType::kBF16>, relu_bwd_supported<DType::kBF16>)
AICF_ELTWISE_FACTORY(make_add_f32_variant, "add_f32_sm100", add_launch<DType::kF32>, add_supported<DType::kF32>)
AICF_ELTWISE_FACTORY(make_add_f16_variant, "add_f16_sm100", add_launch<DType::kF16>, add_supported<DType::kF16>)
AICF_ELTWISE_FACTORY(make_add_bf16_variant, "add_bf16_sm100", add_launch<DType::kBF16>, add_supported<DType::kBF16>)
AICF_ELTWISE_FACTORY(make_mse_grad_f32_variant, "mse_grad_f32_sm100", mse_grad_launch<DType::kF32>, mse_grad_supported<DType::kF32>)
AICF_ELTWISE_FACTORY(make_mse_grad_f16_variant, "mse_grad_f16_sm100", mse_grad_launch<DType::kF16>, mse_grad_supported<DType::kF16>)
AICF_ELTWISE_FACTORY(make_mse_grad_bf16_variant, "mse_grad_bf16_sm100", mse_grad_launch<DType::kBF16>, mse_grad_supported<DType::kBF16>)
AICF_ELTWISE_FACTORY(make_copy_f32_variant, "copy_f32_sm100", copy_launch<DType::kF32>, copy_supported<DType::kF32>)
AICF_ELTWISE_FACTORY(make_copy_f16_variant, "copy_f16_sm100", copy_launch<DType::kF16>, copy_supported<DType::kF16>)
AICF_ELTWISE_FACTORY(make_copy_bf16_variant, "copy_bf16_sm100", copy_launch<DType::kBF16>, copy_supported<DType::kBF16>)
AICF_ELTWISE_FACTORY(make_copy_i32_variant, "copy_i32_sm100", copy_i32_launch, copy_i32_supported)
AICF_ELTWISE_FACTORY(make_grad_zero_variant, "grad_zero_memset", grad_zero_launch, grad_zero_supported)
AICF_ELTWISE_FACTORY(make_bias_add_f32_variant, "bias_add_f32_sm100", bias_add_launch<DType::kF32>, bias_add_supported<DType::kF32>)
AICF_ELTWISE_FACTORY(make_bias_add_f16_variant, "bias_add_f16_sm100", bias_add_launch<DType::kF16>, bias_add_supported<DType::kF16>)
AICF_ELTWISE_FACTORY(make_bias_add_bf16_variant, "bias_add_bf16_sm100", bias_add_launch<DType::kBF16>, bias_add_supported<DType::kBF16>)
AICF_ELTWISE_FACTORY(make_cast_variant, "cast_sm100", cast_launch, cast_supported)

}  // namespace aicf::cuda

// ------------------------------------------------------------------------------------------------
// Stream-mix probe (aicf_b200_stream_probe): the ceiling a streaming kernel with R input and W output arrays can
// reach on this device. It does the least work such a kernel can do - 16-byte evict-first loads of R arrays, one add
// per loaded word, 16-byte evict-first stores of W arrays - with the two launch choices that matter left to the
// caller: packets per array in flight per thread (1, 2 or 4) and 256-thread blocks per SM. The best GB/s over those
// choices is the denominator for kernels with the same stream mix (Adam: 4 reads + 3 writes; an elementwise binary
// op: 2 + 1; a copy: 1 + 1), where a plain copy's rate is not. A measuring aid, not an op.
// ------------------------------------------------------------------------------------------------
namespace aicf::cuda {
namespace {
constexpr int kProbeMaxStreams = 8;
struct ProbeArgs {
  const float4* in[kProbeMaxStreams];
  float4* out[kProbeMaxStreams];
  int64_t packets;
};
template <int R, int W, int U>
__global__ void __launch_bounds__(256) stream_probe_kernel(const ProbeArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < a.packets; i += U * stride) {
    float4 v[U][R];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < R; ++r) v[u][r] = __ldcs(a.in[r] + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float4 s = v[u][0];
#pragma unroll
      for (int r = 1; r < R; ++r) {
        s.x += v[u][r].x; s.y += v[u][r].y; s.z += v[u][r].z; s.w += v[u][r].w;
      }
#pragma unroll
      for (int w = 0; w < W; ++w) __stcs(a.out[w] + i + u * stride, make_float4(s.x + w, s.y, s.z, s.w));
    }
  }
  for (; i < a.packets; i += stride) {
    float4 s = __ldcs(a.in[0] + i);
#pragma unroll
    for (int r = 1; r < R; ++r) {
      const float4 t = __ldcs(a.in[r] + i);
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
#pragma unroll
    for (int w = 0; w < W; ++w) __stcs(a.out[w] + i, make_float4(s.x + w, s.y, s.z, s.w));
  }
}
template <int R, int W>
Status probe_launch(const ProbeArgs& a, int in_flight, int blocks_per_sm, cudaStream_t stream) {
  cudaGetLastError();
  const int grid = streaming_grid(a.packets / in_flight + 1, 256, blocks_per_sm);
  if (in_flight == 1) stream_probe_kernel<R, W, 1><<<grid, 256, 0, stream>>>(a);
  else if (in_flight == 2) stream_probe_kernel<R, W, 2><<<grid, 256, 0, stream>>>(a);
  else stream_probe_kernel<R, W, 4><<<grid, 256, 0, stream>>>(a);
  return launch_status();
}
}  // namespace

// reads in 1..4, writes in 1..3; arrays of `bytes` bytes each (multiple of 16), 16-byte aligned, all distinct;
// in_flight in {1, 2, 4} (0 = 2), blocks_per_sm in 1..1024 (0 = 8; past the resident count the grid is oversubscribed).
Status stream_probe(int reads, int writes, const void* const* in, void* const* out, size_t bytes, int in_flight,
                    int blocks_per_sm, cudaStream_t stream) {
  if (reads < 1 || reads > 4 || writes < 1 || writes > 3 || !in || !out || bytes == 0 || bytes % 16 != 0) return Status::InvalidArgument;
  if (in_flight == 0) in_flight = 2;
  if (blocks_per_sm == 0) blocks_per_sm = 8;
  if ((in_flight != 1 && in_flight != 2 && in_flight != 4) || blocks_per_sm < 1 || blocks_per_sm > 1024) return Status::InvalidArgument;
  ProbeArgs a{};
  for (int r = 0; r < reads; ++r) {
    if (!in[r] || !aligned_to(in[r], 16)) return Status::InvalidArgument;
    a.in[r] = static_cast<const float4*>(in[r]);
  }
  for (int w = 0; w < writes; ++w) {
    if (!out[w] || !aligned_to(out[w], 16)) return Status::InvalidArgument;
    a.out[w] = static_cast<float4*>(out[w]);
  }
  a.packets = static_cast<int64_t>(bytes / 16);
  switch (reads * 4 + writes) {
    case 1 * 4 + 1: return probe_launch<1, 1>(a, in_flight, blocks_per_sm, stream);
    case 1 * 4 + 2: return probe_launch<1, 2>(a, in_flight, blocks_per_sm, stream);
    case 1 * 4 + 3: return probe_launch<1, 3>(a, in_flight, blocks_per_sm, stream);
    case 2 * 4 + 1: return probe_launch<2, 1>(a, in_flight, blocks_per_sm, stream);
    case 2 * 4 + 2: return probe_launch<2, 2>(a, in_flight, blocks_per_sm, stream);
    case 2 * 4 + 3: return probe_launch<2, 3>(a, in_flight, blocks_per_sm, stream);
    case 3 * 4 + 1: return probe_launch<3, 1>(a, in_flight, blocks_per_sm, stream);
    case 3 * 4 + 2: return probe_launch<3, 2>(a, in_flight, blocks_per_sm, stream);
    case 3 * 4 + 3: return probe_launch<3, 3>(a, in_flight, blocks_per_sm, stream);
    case 4 * 4 + 1: return probe_launch<4, 1>(a, in_flight, blocks_per_sm, stream);
    case 4 * 4 + 2: return probe_launch<4, 2>(a, in_flight, blocks_per_sm, stream);
    default: return probe_launch<4, 3>(a, in_flight, blocks_per_sm, stream);
  }
}
}  // namespace aicf::cuda
