from aicf_cuda.core_v2 import lower_to_backend_ops  # noqa: F401
