from aicf_cuda.core_v2 import as_ir_value_obj, get_ir, is_tracing, tracing  # noqa: F401
