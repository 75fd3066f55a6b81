from aicf_cuda.core_v2 import (SymTensor, adam_step, bias_corr, linear, linear_bwd, mse_grad, relu, relu_bwd, save,  # noqa: F401
                               sgd_step, softmax_ce_grad, step_inc, sym_tensor)
