from aicf_cuda.core_v2 import apply_kernel_selection, pick_kernel_id  # noqa: F401
