from aicf_cuda.core_v2 import apply_opt_rules  # noqa: F401
