#pragma once
// Borrowed view of a device tensor handed to kernel variants.
// Field order, sizes and offsets (sizeof == 96) are ABI and equal the reference's
// include/aicf/backends/cuda/registry/tensor_desc.hpp:88-104; static_asserts below pin them.
#include <cstddef>
#include <cstdint>

namespace aicf::cuda {

constexpr int kMaxRank = 4;

enum class DType : uint8_t {
  kUnknown = 0,
  kF32 = 1,
  kF16 = 2,
  kBF16 = 3,
  kI32 = 4,
  // spellings the reference also accepts
  Unknown = kUnknown,
  F32 = kF32,
  F16 = kF16,
  BF16 = kBF16,
  I32 = kI32,
};

constexpr bool dtype_is_known(DType t) { return t != DType::kUnknown; }
constexpr bool dtype_is_float(DType t) {
  return t == DType::kF32 || t == DType::kF16 || t == DType::kBF16;
}
constexpr bool dtype_is_int(DType t) { return t == DType::kI32; }
constexpr bool dtype_is_supported(DType t) {
  return dtype_is_float(t) || dtype_is_int(t) || t == DType::kUnknown;
}
constexpr int32_t dtype_bits(DType t) {
  return (t == DType::kF32 || t == DType::kI32) ? 32 : (t == DType::kF16 || t == DType::kBF16) ? 16 : 0;
}
constexpr int32_t dtype_size_bytes(DType t) { return dtype_bits(t) / 8; }
constexpr const char* dtype_name(DType t) {
  return t == DType::kUnknown ? "unknown"
       : t == DType::kF32     ? "f32"
       : t == DType::kF16     ? "f16"
       : t == DType::kBF16    ? "bf16"
       : t == DType::kI32     ? "i32"
                              : "invalid";
}
// Accumulation type used by contractions and reductions.
constexpr DType dtype_accum_for(DType t) { return t == DType::kI32 ? DType::kI32 : DType::kF32; }

struct TensorDesc {
  void* data = nullptr;          // +0  device pointer, never owned by the callee
  DType dtype = DType::kUnknown; // +8

  union RankND {                 // +12 (named union: the reference keeps it for MSVC)
    int32_t rank;
    int32_t ndim;
    RankND() : rank(0) {}
  } r;

  int64_t shape[kMaxRank] = {0, 0, 0, 0};   // +16 elements
  int64_t stride[kMaxRank] = {0, 0, 0, 0};  // +48 elements, not bytes

  bool contiguous = false;  // +80
  int32_t alignment = 0;    // +84 bytes, 0 = unknown
  int32_t device = 0;       // +88

  int32_t rank() const { return r.rank; }
  bool is_valid_rank() const { return r.rank >= 0 && r.rank <= kMaxRank; }
  bool has_data() const { return data != nullptr; }

  bool has_valid_strides_and_shapes() const {
    if (!is_valid_rank()) return false;
    for (int32_t i = 0; i < r.rank; ++i)
      if (shape[i] <= 0 || stride[i] <= 0) return false;
    return true;  // rank 0 (scalar) has nothing to validate
  }

  // rank 0 is a scalar holding one element.
  int64_t numel() const {
    if (!is_valid_rank()) return 0;
    int64_t n = 1;
    for (int32_t i = 0; i < r.rank; ++i) n *= shape[i];
    return n;
  }
  int64_t nbytes() const { return numel() * static_cast<int64_t>(dtype_size_bytes(dtype)); }

  bool aligned_at_least(int32_t bytes) const {
    if (bytes <= 0) return true;
    return alignment > 0 && alignment >= bytes;  // unknown alignment claims nothing
  }

  bool is_2d() const { return r.rank == 2; }
  bool is_contig_2d_rowmajor() const { return is_2d() && stride[1] == 1 && stride[0] == shape[1]; }
};

static_assert(sizeof(TensorDesc) == 96, "TensorDesc layout is ABI");
static_assert(offsetof(TensorDesc, dtype) == 8 && offsetof(TensorDesc, r) == 12, "TensorDesc layout is ABI");
static_assert(offsetof(TensorDesc, shape) == 16 && offsetof(TensorDesc, stride) == 48, "TensorDesc layout is ABI");
static_assert(offsetof(TensorDesc, contiguous) == 80 && offsetof(TensorDesc, alignment) == 84 &&
              offsetof(TensorDesc, device) == 88, "TensorDesc layout is ABI");

}  // namespace aicf::cuda
