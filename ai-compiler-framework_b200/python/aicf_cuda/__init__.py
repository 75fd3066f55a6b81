"""aicf_cuda: B200 (sm_100a) op backend and captured-plan hot path behind the reference's interfaces.

`aicf_cuda._C` is the drop-in binding module (a compiled pybind11 extension; AICF_BINDING=ctypes selects the
pure-Python ctypes twin `_C_ctypes` instead); `aicf_cuda.Plan` is the C++ captured plan;
`aicf_cuda.Tensor` is a NumPy-only device buffer for callers that do not use torch;
`aicf_cuda.core_v2` is the tracing front end with the reference's names (also importable as `aicf_fw.core_v2`).
"""
import os as _os
import sys as _sys

from ._lib import LIB_PATH, lib  # raises when libaicf_b200.so has not been built: there is no fallback

if _os.environ.get("AICF_BINDING", "").lower() == "ctypes":
    from . import _C_ctypes as _C
    _sys.modules[__name__ + "._C"] = _C
else:
    try:
        from . import _C
    except ImportError as e:  # loud: the extension is part of the product
        raise ImportError(f"aicf_cuda._C (compiled extension) is missing or does not load: {e}. Build it with "
                          "`python ai-compiler-framework_b200/build.py`, or set AICF_BINDING=ctypes to use the "
                          "ctypes module over the same C ABI") from e
from . import core_v2
from .lowering import build_mlp_train_step
from .pipeline import DoubleBufferedStep
from .plan import (ROLE_INPUT, ROLE_PARAM, ROLE_STATIC, Plan, ValueSpec, classify_role, needs_zero_init, pack_attrs,
                   pack_attrs_like_reference_executor, plan_from_json, plan_to_json)
from .tensor import Tensor, bf16_bits_to_f32, f32_to_bf16_bits

__all__ = ["_C", "core_v2", "lib", "LIB_PATH", "Plan", "ValueSpec", "Tensor", "DoubleBufferedStep", "build_mlp_train_step", "pack_attrs",
           "pack_attrs_like_reference_executor", "plan_to_json", "plan_from_json", "classify_role", "needs_zero_init", "f32_to_bf16_bits",
           "bf16_bits_to_f32", "ROLE_INPUT", "ROLE_PARAM", "ROLE_STATIC"]
