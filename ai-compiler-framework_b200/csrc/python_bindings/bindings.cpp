// aicf_cuda._C as a compiled extension module (pybind11, no torch, no CUDA headers): the reference's binding surface
// (src/python_bindings/bindings.cpp:372-548: OpKind, op_call, launch_by_id, trace_enable / trace_reset / trace_get,
// graph_begin / graph_end / graph_launch / graph_reset / graph_stream) over this backend's C ABI (aicf_b200.h).
//
// Tensors are duck-typed: anything with data_ptr(), shape, stride(), dtype and is_contiguous() - a torch.Tensor on a
// CUDA device or an aicf_cuda.Tensor. The descriptor is filled here in C++, so an eager launch costs a few
// attribute look-ups instead of a ctypes structure build per operand. Every non-Ok status raises RuntimeError with
// the library's message, which for the two launch calls is the reference's text
// ("aicf_cuda call failed: kind=<int> (<opname>) status=<Name> (<int>)[ kernel_id=<id>]", :252-258).
//
// This file is compiled by g++ into python/aicf_cuda/_C.<abi tag>.so and linked against libaicf_b200.so (found
// through an $ORIGIN-relative run path); it is not part of that library.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "aicf_b200.h"

namespace py = pybind11;

namespace {

constexpr int kMaxRank = 4;

// Values are ABI (include/aicf/backends/cuda/registry/op_kind.hpp).
enum class OpKind : int {
  EltwiseAdd = 0, EltwiseRelu = 1, Gemm = 2, BiasAdd = 3, ReduceSum = 4, MseGrad = 5, ReluBwd = 6, SgdStep = 7, Copy = 8,
  GradZero = 9, AdamStep = 10, StepInc = 11, BiasCorr = 12, LayerNormFwd = 13, LayerNormBwd = 14, BatchNormFwd = 15,
  BatchNormBwd = 16, GemmEpilogue = 17,
  // additions of this backend
  Softmax = 18, SoftmaxCE = 19, ReduceMax = 20, ReduceMean = 21, AllReduce = 22, Cast = 23, GemmReluBwd = 24, DpAdamStep = 25,
};

[[noreturn]] void raise_last(const char* what, int rc) {
  const char* msg = aicf_b200_last_error();
  if (msg && msg[0]) throw std::runtime_error(msg);
  throw std::runtime_error(std::string(what) + " failed with status " + std::to_string(rc));
}
inline void check(int rc, const char* what) {
  if (rc != AICF_OK) raise_last(what, rc);
}

int dtype_code_from_name(const std::string& n) {
  static const std::unordered_map<std::string, int> kByName = {
      {"f32", 1}, {"float32", 1}, {"torch.float32", 1}, {"torch.float", 1},
      {"f16", 2}, {"float16", 2}, {"torch.float16", 2}, {"torch.half", 2},
      {"bf16", 3}, {"bfloat16", 3}, {"torch.bfloat16", 3},
      {"i32", 4}, {"int32", 4}, {"torch.int32", 4}, {"torch.int", 4}};
  auto it = kByName.find(n);
  return it == kByName.end() ? 0 : it->second;
}

// dtype objects seen so far (torch dtypes are singletons, aicf_cuda.Tensor carries short strings): the string
// conversion happens once per object. The cache holds a reference, so an address is never reused while cached; the
// map itself is never destroyed, because static destructors run after the interpreter is gone and dropping a
// reference then would touch freed memory.
int dtype_code(const py::handle& dtype) {
  static auto* cache = new std::unordered_map<PyObject*, int>();
  auto it = cache->find(dtype.ptr());
  if (it != cache->end()) return it->second;
  const std::string name = py::str(dtype);
  const int code = dtype_code_from_name(name);
  if (code == 0) throw std::runtime_error("dtype must be float16/bfloat16/float32/int32. got: dtype=" + name);
  if (cache->size() < 64) {
    Py_INCREF(dtype.ptr());  // kept for the life of the process
    cache->emplace(dtype.ptr(), code);
  }
  return code;
}

void fill_desc(aicf_tensor_desc& d, const py::handle& t, const char* what) {
  if (t.is_none() || !py::hasattr(t, "data_ptr")) throw std::runtime_error(std::string(what) + ": undefined tensor");
  if (py::hasattr(t, "is_cuda") && !t.attr("is_cuda").cast<bool>())
    throw std::runtime_error(std::string(what) + ": must be CUDA tensor. got: device=cpu dtype=" + std::string(py::str(t.attr("dtype"))));
  const py::tuple shape = py::tuple(t.attr("shape"));
  const int rank = static_cast<int>(shape.size());
  if (rank > kMaxRank)
    throw std::runtime_error(std::string(what) + ": rank out of range. got rank=" + std::to_string(rank) + " (kMaxRank=" +
                             std::to_string(kMaxRank) + ")");
  const py::tuple stride = py::tuple(t.attr("stride")());
  d = aicf_tensor_desc{};
  d.data = reinterpret_cast<void*>(t.attr("data_ptr")().cast<uintptr_t>());
  d.dtype = static_cast<uint8_t>(dtype_code(t.attr("dtype")));
  d.rank = rank;
  for (int i = 0; i < rank; ++i) {
    d.shape[i] = shape[i].cast<int64_t>();
    d.stride[i] = stride[i].cast<int64_t>();
  }
  d.contiguous = t.attr("is_contiguous")().cast<bool>() ? 1 : 0;
  d.alignment = 0;  // unknown, as the reference's binding passes it (:122)
  d.device = 0;
}

std::vector<aicf_tensor_desc> build_descs(const py::sequence& seq, const char* what) {
  std::vector<aicf_tensor_desc> v(py::len(seq));
  size_t i = 0;
  for (const py::handle t : seq) fill_desc(v[i++], t, what);
  return v;
}

// All-empty attrs travel as a null blob, like the reference (:303-304).
struct Attrs {
  std::string bytes;
  aicf_attr_blob blob{};
  const aicf_attr_blob* ptr = nullptr;
  Attrs(uint32_t schema_id, const py::bytes& payload) : bytes(payload) {
    if (schema_id == 0 && bytes.empty()) return;
    blob.schema_id = schema_id;
    blob.bytes = static_cast<uint32_t>(bytes.size());
    blob.data = bytes.empty() ? nullptr : bytes.data();
    ptr = &blob;
  }
};

int kind_of(const py::handle& kind) {
  if (py::isinstance<OpKind>(kind)) return static_cast<int>(kind.cast<OpKind>());
  return kind.cast<int>();
}

void op_call(const py::object& kind, const py::sequence& inputs, const py::sequence& outputs, uint32_t schema_id,
             const py::bytes& attrs_bytes, uint64_t stream) {
  auto in = build_descs(inputs, "inputs");
  auto out = build_descs(outputs, "outputs");
  const Attrs a(schema_id, attrs_bytes);
  check(aicf_b200_op_call_traced(kind_of(kind), in.data(), static_cast<int>(in.size()), out.data(), static_cast<int>(out.size()),
                                 a.ptr, stream),
        "op_call");
}

void launch_by_id(const std::string& kernel_id, const py::object& kind, const py::sequence& inputs, const py::sequence& outputs,
                  uint32_t schema_id, const py::bytes& attrs_bytes, uint64_t stream) {
  auto in = build_descs(inputs, "inputs");
  auto out = build_descs(outputs, "outputs");
  const Attrs a(schema_id, attrs_bytes);
  check(aicf_b200_launch_by_id_traced(kernel_id.c_str(), kind_of(kind), in.data(), static_cast<int>(in.size()), out.data(),
                                      static_cast<int>(out.size()), a.ptr, stream),
        "launch_by_id");
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "aicf_cuda._C: op dispatch, op trace and the process-wide CUDA graph of the B200 backend";
  m.attr("binding") = "pybind11";

  py::enum_<OpKind>(m, "OpKind", py::arithmetic())
      .value("EltwiseAdd", OpKind::EltwiseAdd).value("EltwiseRelu", OpKind::EltwiseRelu).value("Gemm", OpKind::Gemm)
      .value("BiasAdd", OpKind::BiasAdd).value("ReduceSum", OpKind::ReduceSum).value("MseGrad", OpKind::MseGrad)
      .value("ReluBwd", OpKind::ReluBwd).value("SgdStep", OpKind::SgdStep).value("Copy", OpKind::Copy)
      .value("GradZero", OpKind::GradZero).value("AdamStep", OpKind::AdamStep).value("StepInc", OpKind::StepInc)
      .value("BiasCorr", OpKind::BiasCorr).value("LayerNormFwd", OpKind::LayerNormFwd).value("LayerNormBwd", OpKind::LayerNormBwd)
      .value("BatchNormFwd", OpKind::BatchNormFwd).value("BatchNormBwd", OpKind::BatchNormBwd)
      .value("GemmEpilogue", OpKind::GemmEpilogue).value("Softmax", OpKind::Softmax).value("SoftmaxCE", OpKind::SoftmaxCE)
      .value("ReduceMax", OpKind::ReduceMax).value("ReduceMean", OpKind::ReduceMean).value("AllReduce", OpKind::AllReduce)
      .value("Cast", OpKind::Cast).value("GemmReluBwd", OpKind::GemmReluBwd).value("DpAdamStep", OpKind::DpAdamStep)
      .export_values();

  m.def("op_call", &op_call, py::arg("kind"), py::arg("inputs"), py::arg("outputs"), py::arg("schema_id") = 0,
        py::arg("attrs_bytes") = py::bytes(""), py::arg("stream") = 0,
        "Legacy runtime dispatch: the first kernel variant that supports the operands runs.");
  m.def("launch_by_id", &launch_by_id, py::arg("kernel_id"), py::arg("kind"), py::arg("inputs"), py::arg("outputs"),
        py::arg("schema_id") = 0, py::arg("attrs_bytes") = py::bytes(""), py::arg("stream") = 0,
        "Decision-applied path: runs exactly the variant registered under kernel_id.");

  m.def("trace_enable", [](bool flag) { aicf_b200_trace_enable(flag ? 1 : 0); }, py::arg("flag") = true);
  m.def("trace_reset", [] { aicf_b200_trace_reset(); });
  m.def("trace_get", [] {
    std::vector<std::string> out;
    const int n = aicf_b200_trace_count();
    for (int i = 0; i < n; ++i) {
      const char* s = aicf_b200_trace_get(i);
      if (!s) break;
      out.emplace_back(s);
    }
    return out;
  });

  m.def("graph_begin", [] {
    uint64_t s = 0;
    check(aicf_b200_graph_begin(&s), "graph_begin");
    return s;
  });
  m.def("graph_end", [] { check(aicf_b200_graph_end(), "graph_end"); });
  m.def("graph_launch", [] { check(aicf_b200_graph_launch(), "graph_launch"); });
  m.def("graph_reset", [] { check(aicf_b200_graph_reset(), "graph_reset"); });
  m.def("graph_stream", [] { return aicf_b200_graph_stream(); });

  // ---- additions (not in the reference module) ----
  m.def("kernel_ids", [](const py::object& kind) {
    std::vector<std::string> out;
    const int k = kind_of(kind), n = aicf_b200_kernel_count(k);
    for (int i = 0; i < n; ++i) out.emplace_back(aicf_b200_kernel_id(k, i));
    return out;
  }, py::arg("kind"), "Registered kernel ids of an op kind, in dispatch priority order.");
  m.def("gemm_status", [](bool clear) { return aicf_b200_gemm_status(clear ? 1 : 0); }, py::arg("clear") = false,
        "0 unless a bounded wait inside the tcgen05 GEMM expired; synchronises the device.");
  m.def("wait_status", [](bool clear) { return aicf_b200_wait_status(clear ? 1 : 0); }, py::arg("clear") = false,
        "0 unless a bounded device-side wait expired (GEMM pipeline, row prefetch, exchange); synchronises the device.");
  m.def("device_sync", [] { check(aicf_b200_device_sync(), "device_sync"); });
}
