from aicf_cuda.core_v2 import ExecOptions, PlannedExecutor, opkind_from_name  # noqa: F401
