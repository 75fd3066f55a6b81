"""CPU oracle for the op backend: TEST INFRASTRUCTURE ONLY.

A NumPy restatement of what each lowered op computes, used to check the CUDA kernels and as the
timed CPU baseline of bench.py. Nothing in the shipped package imports this directory; the product
path has no CPU fallback.

Pinning status. The reference ships no golden tensors and no asserting numeric tests (its probe
scripts print max|delta| against torch), and it has no CPU implementation. So:
  * ops the reference implements (gemm, gemm_epilogue, bias_add, relu, relu_bwd, copy, grad_zero,
    mse_grad, reduce_sum column sum, adam_step, step_inc, bias_corr, sgd_step, add, layernorm_fwd,
    layernorm_bwd; f32 and f16) are pinned twice: on a GPU machine by running the reference's own CUDA
    sources, compiled unmodified into oracle/_ref/ (see ref_build.py), on the same device buffers -
    tests/test_ref_parity.py, tests/test_layernorm_gpu.py; and on any machine against the outputs of
    those kernels stored in tests/golden/ref_cuda_golden.npz - tests/test_oracle_cpu.py;
  * softmax, softmax_ce, last-axis sum/max/mean, every bf16 variant, Adam weight decay and the
    fused-step Adam do not exist in the reference: for those, PARITY IS UNPINNED by the reference and
    the fp64 restatement of the published definitions below is the only oracle.
Structural fixtures the reference does commit (lowered-op list, binding-plan roles, runtime trace
strings) are checked in tests/test_boundary_fixture.py.
"""
from .ops import *  # noqa: F401,F403
from .interp import run_lowered  # noqa: F401
from .inputs import *  # noqa: F401,F403
