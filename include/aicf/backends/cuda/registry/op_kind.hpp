#pragma once
// Operation kinds. Values 0..17 are ABI shared with the reference
// (include/aicf/backends/cuda/registry/op_kind.hpp:5-31); kinds from 18 up are
// additions of this backend and are only ever appended.

namespace aicf::cuda {

enum class OpKind : int {
  EltwiseAdd = 0,
  EltwiseRelu = 1,
  Gemm = 2,
  BiasAdd = 3,
  ReduceSum = 4,
  MseGrad = 5,
  ReluBwd = 6,
  SgdStep = 7,
  Copy = 8,
  GradZero = 9,
  AdamStep = 10,
  StepInc = 11,
  BiasCorr = 12,
  LayerNormFwd = 13,
  LayerNormBwd = 14,
  BatchNormFwd = 15,
  BatchNormBwd = 16,
  GemmEpilogue = 17,

  // ---- additions (not present in the reference) ----
  Softmax = 18,     // row softmax over the last axis
  SoftmaxCE = 19,   // fused softmax cross-entropy: loss rows, gradient, argmax
  ReduceMax = 20,   // last-axis max
  ReduceMean = 21,  // last-axis mean
  AllReduce = 22,   // in-place sum over data-parallel ranks
  Cast = 23,        // dtype conversion (f32 <-> bf16/f16)
  GemmReluBwd = 24, // dX = (Y > 0) ? dY * op(W) : 0  (the ReLU backward mask applied in the GEMM epilogue)

  DpAdamStep = 25,  // data-parallel Adam fused with its gradient exchange over peer memory

  _Count = 26,
  // Number of kinds the reference defines; ids below this resolve exactly as there.
  _ReferenceCount = 18
};

// Lower-case op name used in traces and lowered-op lists
// (reference: src/python_bindings/bindings.cpp:196-219).
inline const char* op_kind_name(OpKind k) {
  switch (k) {
    case OpKind::EltwiseAdd: return "add";
    case OpKind::EltwiseRelu: return "relu";
    case OpKind::Gemm: return "gemm";
    case OpKind::BiasAdd: return "bias_add";
    case OpKind::ReduceSum: return "reduce_sum";
    case OpKind::MseGrad: return "mse_grad";
    case OpKind::ReluBwd: return "relu_bwd";
    case OpKind::SgdStep: return "sgd_step";
    case OpKind::Copy: return "copy";
    case OpKind::GradZero: return "grad_zero";
    case OpKind::AdamStep: return "adam_step";
    case OpKind::StepInc: return "step_inc";
    case OpKind::BiasCorr: return "bias_corr";
    case OpKind::LayerNormFwd: return "layernorm_fwd";
    case OpKind::LayerNormBwd: return "layernorm_bwd";
    case OpKind::BatchNormFwd: return "batchnorm_fwd";
    case OpKind::BatchNormBwd: return "batchnorm_bwd";
    case OpKind::GemmEpilogue: return "gemm_epilogue";
    case OpKind::Softmax: return "softmax";
    case OpKind::SoftmaxCE: return "softmax_ce";
    case OpKind::ReduceMax: return "reduce_max";
    case OpKind::ReduceMean: return "reduce_mean";
    case OpKind::AllReduce: return "all_reduce";
    case OpKind::Cast: return "cast";
    case OpKind::GemmReluBwd: return "gemm_relu_bwd";
    case OpKind::DpAdamStep: return "dp_adam_step";
    default: return "unknown";
  }
}

}  // namespace aicf::cuda
