#pragma once
// Registers every kernel variant of this backend. Idempotence is the caller's job
// (KernelRegistry::ensure_registered wraps it in call_once), as in the reference
// (register_all.hpp:8, register_all.cpp:88-291).
#ifdef __cplusplus
extern "C" {
#endif
void aicf_cuda_register_all_kernels();
#ifdef __cplusplus
}
#endif
