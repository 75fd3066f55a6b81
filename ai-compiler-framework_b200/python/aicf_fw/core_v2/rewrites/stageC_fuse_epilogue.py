from aicf_cuda.core_v2 import stageC_fuse_gemm_epilogue  # noqa: F401
