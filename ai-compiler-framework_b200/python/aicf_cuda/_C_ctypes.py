"""The binding surface of the reference's pybind/torch extension over the C ABI, in pure Python (ctypes).

`aicf_cuda._C` is normally the compiled extension module (csrc/python_bindings/bindings.cpp, built by build.py), which
offers exactly these names. This module is the alternative for an interpreter the extension was not built for:
AICF_BINDING=ctypes in the environment makes `aicf_cuda._C` resolve to it. Both go through the same C entry points
(aicf_b200_op_call_traced / aicf_b200_launch_by_id_traced), so traces, error texts and results are identical; the
compiled module only spends less host time per eager launch.

Same names, argument order, defaults, trace strings and error texts as the reference module
(src/python_bindings/bindings.cpp:372-548): OpKind, op_call, launch_by_id, trace_enable/reset/get,
graph_begin/end/launch/reset/stream. Tensors are duck-typed: torch.Tensor (CUDA), aicf_cuda.Tensor or
anything exposing data_ptr() / shape / stride() / dtype. bf16 is accepted in addition to the
reference's f16 / f32 / i32.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Any, Sequence

from ._lib import AttrBlob, TensorDesc, check, lib

_K_MAX_RANK = 4


class OpKind(enum.IntEnum):
    EltwiseAdd = 0
    EltwiseRelu = 1
    Gemm = 2
    BiasAdd = 3
    ReduceSum = 4
    MseGrad = 5
    ReluBwd = 6
    SgdStep = 7
    Copy = 8
    GradZero = 9
    AdamStep = 10
    StepInc = 11
    BiasCorr = 12
    LayerNormFwd = 13
    LayerNormBwd = 14
    BatchNormFwd = 15
    BatchNormBwd = 16
    GemmEpilogue = 17
    # additions of this backend
    Softmax = 18
    SoftmaxCE = 19
    ReduceMax = 20
    ReduceMean = 21
    AllReduce = 22
    Cast = 23
    GemmReluBwd = 24
    DpAdamStep = 25


# pybind's export_values(): enumerators are also module attributes
globals().update(OpKind.__members__)
binding = "ctypes"

_DTYPE_BY_NAME = {
    "f32": 1, "float32": 1, "torch.float32": 1, "torch.float": 1,
    "f16": 2, "float16": 2, "torch.float16": 2, "torch.half": 2,
    "bf16": 3, "bfloat16": 3, "torch.bfloat16": 3,
    "i32": 4, "int32": 4, "torch.int32": 4, "torch.int": 4,
}


def _dtype_code(t: Any) -> int:
    name = str(getattr(t, "dtype", None))
    code = _DTYPE_BY_NAME.get(name)
    if code is None:
        raise RuntimeError(f"dtype must be float16/bfloat16/float32/int32. got: dtype={name}")
    return code


def _fill_desc(d: TensorDesc, t: Any, what: str) -> None:
    if t is None or not hasattr(t, "data_ptr"):
        raise RuntimeError(f"{what}: undefined tensor")
    if hasattr(t, "is_cuda") and not t.is_cuda:
        raise RuntimeError(f"{what}: must be CUDA tensor. got: device=cpu dtype={t.dtype}")
    shape = tuple(int(s) for s in t.shape)
    rank = len(shape)
    if rank > _K_MAX_RANK:
        raise RuntimeError(f"{what}: rank out of range. got rank={rank} (kMaxRank={_K_MAX_RANK})")
    stride = tuple(int(s) for s in t.stride())
    d.data = int(t.data_ptr())
    d.dtype = _dtype_code(t)
    d.rank = rank
    for i in range(rank):
        d.shape[i] = shape[i]
        d.stride[i] = stride[i]
    d.contiguous = 1 if t.is_contiguous() else 0
    d.alignment = 0
    d.device = 0


def _build_descs(seq: Sequence[Any], what: str):
    n = len(seq)
    arr = (TensorDesc * max(n, 1))()
    for i, t in enumerate(seq):
        _fill_desc(arr[i], t, what)
    return arr, n


def _blob(schema_id: int, attrs_bytes: bytes):
    """Returns (blob pointer or None, keep-alive). All-empty attrs are passed as a null blob."""
    attrs_bytes = bytes(attrs_bytes or b"")
    if schema_id == 0 and not attrs_bytes:
        return None, None
    buf = C.create_string_buffer(attrs_bytes, len(attrs_bytes)) if attrs_bytes else None
    b = AttrBlob(int(schema_id) & 0xFFFFFFFF, len(attrs_bytes), C.cast(buf, C.c_void_p) if buf else None)
    return C.byref(b), (b, buf)


def op_call(kind, inputs, outputs, schema_id: int = 0, attrs_bytes: bytes = b"", stream: int = 0) -> None:
    """Legacy runtime dispatch: the first kernel variant that supports the operands runs."""
    ins, ni = _build_descs(inputs, "inputs")
    outs, no = _build_descs(outputs, "outputs")
    blob, _keep = _blob(schema_id, attrs_bytes)
    check(lib.aicf_b200_op_call_traced(int(kind), ins, ni, outs, no, blob, int(stream)), "op_call")


def launch_by_id(kernel_id: str, kind, inputs, outputs, schema_id: int = 0, attrs_bytes: bytes = b"",
                 stream: int = 0) -> None:
    """Decision-applied path: runs exactly the variant registered under `kernel_id`."""
    ins, ni = _build_descs(inputs, "inputs")
    outs, no = _build_descs(outputs, "outputs")
    blob, _keep = _blob(schema_id, attrs_bytes)
    check(lib.aicf_b200_launch_by_id_traced(str(kernel_id).encode(), int(kind), ins, ni, outs, no, blob, int(stream)),
          "launch_by_id")


def trace_enable(flag: bool = True) -> None:
    lib.aicf_b200_trace_enable(1 if flag else 0)


def trace_reset() -> None:
    lib.aicf_b200_trace_reset()


def trace_get() -> list[str]:
    out = []
    for i in range(lib.aicf_b200_trace_count()):
        s = lib.aicf_b200_trace_get(i)
        if s is None:
            break
        out.append(s.decode())
    return out


def graph_begin() -> int:
    s = C.c_uint64(0)
    check(lib.aicf_b200_graph_begin(C.byref(s)), "graph_begin")
    return int(s.value)


def graph_end() -> None:
    check(lib.aicf_b200_graph_end(), "graph_end")


def graph_launch() -> None:
    check(lib.aicf_b200_graph_launch(), "graph_launch")


def graph_reset() -> None:
    check(lib.aicf_b200_graph_reset(), "graph_reset")


def graph_stream() -> int:
    return int(lib.aicf_b200_graph_stream())


# ---- additions (not in the reference module) ------------------------------------------------------
def kernel_ids(kind) -> list[str]:
    """Registered kernel ids of an op kind, in dispatch priority order."""
    return [lib.aicf_b200_kernel_id(int(kind), i).decode() for i in range(lib.aicf_b200_kernel_count(int(kind)))]


def gemm_status(clear: bool = False) -> int:
    """0 unless a bounded wait inside the tcgen05 GEMM expired; synchronises the device."""
    return int(lib.aicf_b200_gemm_status(1 if clear else 0))


def wait_status(clear: bool = False) -> int:
    """0 unless a bounded device-side wait expired (GEMM pipeline or softmax row prefetch); synchronises."""
    return int(lib.aicf_b200_wait_status(1 if clear else 0))


def device_sync() -> None:
    check(lib.aicf_b200_device_sync(), "device_sync")
