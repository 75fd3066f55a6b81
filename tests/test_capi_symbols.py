"""The C-ABI library loads on a machine without a GPU and exports every symbol include/aicf_b200.h
declares; the ctypes prototype table covers the same set."""
import re
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (REPO / "include" / "aicf_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(aicf_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    assert len(names) >= 60
    for must in ("aicf_b200_op_call", "aicf_b200_launch_by_id", "aicf_b200_graph_begin", "aicf_b200_plan_capture",
                 "aicf_b200_plan_replay", "aicf_b200_dp_init"):
        assert must in names


def test_library_exports_every_declared_symbol():
    import aicf_cuda
    for name in declared_functions():
        assert hasattr(aicf_cuda.lib, name), f"{name} declared in aicf_b200.h but not exported"


def test_ctypes_table_matches_header():
    from aicf_cuda._lib import PROTOTYPES
    assert sorted(PROTOTYPES) == declared_functions()


def test_abi_version_and_status_strings():
    import aicf_cuda
    lib = aicf_cuda.lib
    assert lib.aicf_b200_abi_version() == 1
    assert [lib.aicf_b200_status_string(i).decode() for i in range(5)] == ["Ok", "InvalidArgument", "NotImplemented", "Internal", "Unknown"]


def test_op_names_follow_the_reference_binding():
    import aicf_cuda
    want = ["add", "relu", "gemm", "bias_add", "reduce_sum", "mse_grad", "relu_bwd", "sgd_step", "copy", "grad_zero",
            "adam_step", "step_inc", "bias_corr", "layernorm_fwd", "layernorm_bwd", "batchnorm_fwd", "batchnorm_bwd",
            "gemm_epilogue", "softmax", "softmax_ce", "reduce_max", "reduce_mean", "all_reduce", "cast", "gemm_relu_bwd", "dp_adam_step"]
    got = [aicf_cuda.lib.aicf_b200_op_name(i).decode() for i in range(len(want))]
    assert got == want
    assert aicf_cuda.lib.aicf_b200_op_name(99).decode() == "unknown"


def test_opkind_enum_values_are_abi():
    from aicf_cuda._C import OpKind
    assert [int(OpKind.EltwiseAdd), int(OpKind.Gemm), int(OpKind.AdamStep), int(OpKind.GemmEpilogue)] == [0, 2, 10, 17]
    import aicf_cuda._C as m
    assert m.Gemm == OpKind.Gemm  # export_values()
    assert OpKind(17) == OpKind.GemmEpilogue and int(OpKind(17)) == 17


def test_compiled_and_ctypes_binding_modules_offer_the_same_surface():
    """aicf_cuda._C is the compiled extension by default; _C_ctypes is its pure-Python twin over the same C ABI."""
    import aicf_cuda
    import aicf_cuda._C as native
    import aicf_cuda._C_ctypes as twin
    import os
    expected = "ctypes" if os.environ.get("AICF_BINDING", "").lower() == "ctypes" else "pybind11"
    assert native.binding == expected and twin.binding == "ctypes" and aicf_cuda._C is native
    names = ["OpKind", "op_call", "launch_by_id", "trace_enable", "trace_reset", "trace_get", "graph_begin", "graph_end",
             "graph_launch", "graph_reset", "graph_stream", "kernel_ids", "gemm_status", "wait_status", "device_sync"]
    for n in names:
        assert hasattr(native, n) and hasattr(twin, n), n
    assert {k: int(v) for k, v in native.OpKind.__members__.items()} == {k: int(v) for k, v in twin.OpKind.__members__.items()}
    assert native.kernel_ids(native.OpKind.Copy) == twin.kernel_ids(twin.OpKind.Copy)
    # the reference's error texts, from either module, without a device
    import pytest
    for mod in (native, twin):
        with pytest.raises(RuntimeError, match="graph_end called but not capturing"):
            mod.graph_end()
        with pytest.raises(RuntimeError, match="graph_launch called but no captured graph exists"):
            mod.graph_launch()
        with pytest.raises(RuntimeError, match=r"aicf_cuda call failed: kind=2 \(gemm\) status=NotImplemented \(2\) kernel_id=nope_v0"):
            mod.launch_by_id("nope_v0", mod.OpKind.Gemm, [], [])

        class Fake:
            dtype, shape = "f64", (2, 2)
            def data_ptr(self): return 4096
            def stride(self): return (2, 1)
            def is_contiguous(self): return True
        with pytest.raises(RuntimeError, match="dtype must be float16/bfloat16/float32/int32"):
            mod.op_call(mod.OpKind.EltwiseRelu, [Fake()], [Fake()])
        Fake.dtype, Fake.shape = "f32", (1, 1, 1, 1, 1)
        with pytest.raises(RuntimeError, match="rank out of range"):
            mod.op_call(mod.OpKind.EltwiseRelu, [Fake()], [Fake()])
        mod.trace_reset()
        mod.trace_enable(True)
        assert mod.trace_get() == []


def test_null_pointer_calls_fail_cleanly_without_a_device():
    import aicf_cuda
    lib = aicf_cuda.lib
    # by-id with no id -> InvalidArgument; unknown id -> NotImplemented; both without touching the GPU
    assert lib.aicf_b200_launch_by_id(None, 2, None, 0, None, 0, None, 0) == 1
    assert lib.aicf_b200_launch_by_id(b"no_such_kernel_v0", 2, None, 0, None, 0, None, 0) == 2
    assert "kernel_id=no_such_kernel_v0" in lib.aicf_b200_last_error().decode()
    assert lib.aicf_b200_launch_by_id(b"batchnorm_fwd_f16_v0", 15, None, 0, None, 0, None, 0) == 2   # not registered
    assert lib.aicf_b200_op_call(99, None, 0, None, 0, None, 0) == 1
    assert lib.aicf_b200_graph_end() == 1
    assert lib.aicf_b200_last_error().decode() == "graph_end called but not capturing"
    assert lib.aicf_b200_graph_launch() == 1
    assert lib.aicf_b200_last_error().decode() == "graph_launch called but no captured graph exists"


def test_binding_survives_interpreter_exit_with_cached_runtime_dtype_objects():
    """The compiled module caches dtype objects it has seen. A dtype that is an ordinary run-time string (not an
    interned constant) must not be released from a C++ static destructor after the interpreter is gone."""
    import subprocess
    import sys
    from pathlib import Path
    repo = Path(__file__).resolve().parents[1]
    code = (
        "import sys; sys.path.insert(0, 'ai-compiler-framework_b200/python')\n"
        "from aicf_cuda import _C\n"
        "class T:\n"
        "    def __init__(s, dt): s.dtype, s.shape = dt, (2, 2)\n"
        "    def data_ptr(s): return 4096\n"
        "    def stride(s): return (2, 1)\n"
        "    def is_contiguous(s): return True\n"
        "for dt in [''.join(['f', '3', '2']), ''.join(['b', 'f', '1', '6'])]:\n"
        "    try: _C.launch_by_id('nope_v0', _C.OpKind.EltwiseRelu, [T(dt)], [T(dt)])\n"
        "    except RuntimeError: pass\n"
        "print('DONE')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(repo), timeout=120)
    assert r.returncode == 0 and "DONE" in r.stdout, f"exit code {r.returncode}\n{r.stderr[-500:]}"
