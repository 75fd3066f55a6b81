from aicf_cuda.core_v2 import trace_ir  # noqa: F401
