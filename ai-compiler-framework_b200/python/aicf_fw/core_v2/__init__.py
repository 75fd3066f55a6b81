"""Same names as the reference's python/aicf_fw/core_v2/__init__.py, served by aicf_cuda.core_v2."""
from aicf_cuda.core_v2 import (BindingPlan, ExecOptions, PlannedExecutor, PlanOptions, SymTensor, build_binding_plan, dump_ir,
                               dump_lowered, dump_plan, linear, lower_to_backend_ops, mse_grad, relu, sym_tensor, trace_ir)

__all__ = ["trace_ir", "dump_ir", "dump_lowered", "dump_plan", "lower_to_backend_ops", "build_binding_plan", "BindingPlan",
           "PlanOptions", "SymTensor", "sym_tensor", "linear", "relu", "mse_grad", "PlannedExecutor", "ExecOptions"]
