from aicf_cuda.core_v2 import (ROLE_INPUT, ROLE_PARAM, ROLE_STATIC, BindingPlan, BindSpec, PlanOptions,  # noqa: F401
                               apply_kernel_decisions_stageB, build_binding_plan)
