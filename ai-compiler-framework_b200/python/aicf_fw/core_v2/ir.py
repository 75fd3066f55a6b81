from aicf_cuda.core_v2 import IRGraph, IRNode, IRValue  # noqa: F401
