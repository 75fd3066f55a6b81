#pragma once
// Registers every kernel variant of this backend with KernelRegistry::instance(). C linkage, so that a host
// written in another language (or a dlopen'ing loader) can find it by its plain name. Calling it twice registers
// nothing new (the first registration of a kernel id wins) but is wasted work: KernelRegistry::ensure_registered()
// wraps it in std::call_once and is what dispatch uses. Same symbol and contract as the reference's
// register_all.hpp:8 / register_all.cpp:88-291.
#if defined(__cplusplus)
#define AICF_CUDA_C_LINKAGE extern "C"
#else
#define AICF_CUDA_C_LINKAGE
#endif

AICF_CUDA_C_LINKAGE void aicf_cuda_register_all_kernels();
