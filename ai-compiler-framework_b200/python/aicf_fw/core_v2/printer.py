from aicf_cuda.core_v2 import dump_ir, dump_lowered, dump_plan  # noqa: F401
