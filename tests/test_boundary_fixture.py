"""The reference's committed boundary dumps (lowered-op list, binding-plan roles, runtime trace) as a
fixture: ids resolve, roles classify the same way, the trace reproduces string for string."""
import json
from pathlib import Path

import numpy as np
import pytest

import aicf_cuda
from aicf_cuda import _C, Plan, Tensor, ValueSpec, classify_role, pack_attrs, pack_attrs_like_reference_executor
from aicf_cuda._C import OpKind

FIX = json.loads((Path(__file__).resolve().parent / "golden" / "boundary_fixture.json").read_text())

OPNAME_TO_KIND = {
    "add": 0, "relu": 1, "gemm": 2, "bias_add": 3, "reduce_sum": 4, "mse_grad": 5, "relu_bwd": 6, "sgd_step": 7,
    "copy": 8, "copy_saved": 8, "copy_aux": 8, "grad_zero": 9, "adam_step": 10, "step_inc": 11, "bias_corr": 12,
    "gemm_epilogue": 17,
}

# kernel ids of the reference's MLP path (its register_all.cpp); all must stay resolvable
REFERENCE_IDS = {
    4: ["reduce_sum_keep_lastdim_f16_v0", "reduce_sum_keep_lastdim_f16_to_f32_v0", "reduce_sum_keep_lastdim_f32_v0"],
    2: ["gemm_f16_tc_wmma_out_f16_v0", "gemm_f32_naive_v0"],
    17: ["gemm_bias_relu_f16_tc_wmma_out_f16_v0", "gemm_bias_relu_f32_naive_v0"],
    3: ["bias_add_f16_vec2_v0", "bias_add_f16_v0", "bias_add_f32_v0"],
    0: ["add_f16_vec2_v0", "add_f16_v0", "add_f32_v0"],
    1: ["relu_f16_vec2_v0", "relu_f16_v0", "relu_f32_v0"],
    5: ["mse_grad_f16_v0", "mse_grad_f32_v0"],
    6: ["relu_bwd_f16_vec2_v0", "relu_bwd_f16_v0", "relu_bwd_f32_v0"],
    7: ["sgd_step_f16_half2_v0", "sgd_step_f16_v0", "sgd_step_f32_v0"],
    8: ["copy_f16_v0", "copy_f32_v0"],
    9: ["grad_zero_v0"],
    10: ["adam_step_f32_v0"],
    11: ["step_inc_v0"],
    12: ["bias_corr_v0"],
}


def test_reference_kernel_ids_resolve_in_reference_priority_order():
    for kind, ids in REFERENCE_IDS.items():
        ours = _C.kernel_ids(kind)
        for kid in ids:
            assert kid in ours, f"{kid} missing from kind {kind}"
        kept = [k for k in ours if k in ids]
        assert kept == ids, f"relative dispatch order changed for kind {kind}: {kept}"


def test_fixture_ids_are_registered_under_the_fixture_kinds():
    for it in FIX["lowered"]:
        assert it["kernel_id"] in _C.kernel_ids(OPNAME_TO_KIND[it["op"]])


def test_roles_classify_like_the_reference_binding_plan():
    role_name = {0: "input", 1: "param", 2: "static"}
    for v in FIX["values"]:
        assert role_name[classify_role(v["name"])] == v["role"], v["name"]
    assert sum(v["role"] == "input" for v in FIX["values"]) == 2
    assert sum(v["role"] == "param" for v in FIX["values"]) == 4


def test_trace_strings_derive_from_the_lowered_list():
    want = [f"kid:{it['kernel_id']} kind:{aicf_cuda.lib.aicf_b200_op_name(OPNAME_TO_KIND[it['op']]).decode()}"
            for it in FIX["lowered"]]
    assert want == FIX["runtime_trace"]


def test_attr_packing_matches_both_contracts():
    assert pack_attrs("gemm", {"transB": True}) == (0x47454D4D, b"\x00\x00\x00\x00\x01\x00\x00\x00")
    assert pack_attrs("gemm_epilogue", {"epilogue_act": "relu", "epilogue_bias": True, "transB": True}) == (
        0x4750454C, b"\x00\x00\x00\x00\x01\x00\x00\x00\x01\x00\x00\x00")
    assert pack_attrs("gemm_epilogue", {"epilogue": "bias"})[1][8:] == b"\x00\x00\x00\x00"
    assert pack_attrs("sgd_step", {"lr": 0.01})[0] == 0x53444753
    assert pack_attrs("reduce_sum", {"axis": 0, "keepdim": False}) == (0x5253554D, b"\x00" * 8)
    assert pack_attrs("bias_corr", {})[0] == 0x524F4342
    assert pack_attrs("relu", {}) == (0, b"")
    # the reference's executor: schema 0 for gemm, 'GEPI' for the epilogue, nothing for sgd/reduce
    assert pack_attrs_like_reference_executor("gemm", {"transB": True})[0] == 0
    assert pack_attrs_like_reference_executor("gemm_epilogue", {})[0] == int.from_bytes(b"GEPI", "little")
    assert pack_attrs_like_reference_executor("sgd_step", {"lr": 0.01}) == (0, b"")


def test_plan_json_round_trip_keeps_the_lowered_contract():
    from aicf_cuda import build_mlp_train_step, plan_from_json, plan_to_json
    vals, low = build_mlp_train_step(64, [784, 256, 10], compute_dtype="bf16", data_parallel="fused", weight_decay=0.01)
    text = plan_to_json("mlp", vals, low)
    name, vals2, low2 = plan_from_json(text)
    assert name == "mlp" and plan_to_json(name, vals2, low2) == text
    assert [(v.vid, v.name, v.shape, v.dtype, v.peer_visible) for v in vals2] == [(v.vid, v.name, v.shape, v.dtype, v.peer_visible) for v in vals]
    assert [it["op"] for it in low2] == [it["op"] for it in low] and low2[2]["kernel_id"] == low[2]["kernel_id"]
    assert [pack_attrs(it["op"], it["attrs"]) for it in low2] == [pack_attrs(it["op"], it["attrs"]) for it in low]
    # the reference's own lowered list (fixture) survives the same trip
    fvals = [ValueSpec(v["vid"], v["name"], tuple(v["shape"]), _TORCH_DT[v["dtype"]]) for v in FIX["values"]]
    _, _, flow = plan_from_json(plan_to_json("fixture", fvals, FIX["lowered"]))
    assert flow == FIX["lowered"]
    with pytest.raises(ValueError):
        plan_from_json('{"format": "something else"}')


_TORCH_DT = {"float16": "f16", "float32": "f32", "int32": "i32"}


def _fixture_inputs():
    rng = np.random.default_rng(0)
    out = {}
    for v in FIX["values"]:
        if v["role"] in ("input", "param"):
            out[v["vid"]] = (rng.standard_normal(v["shape"]) * 0.5).astype(np.float16)
    return out


@pytest.mark.gpu
def test_eager_launch_by_id_reproduces_the_runtime_trace_and_the_oracle(gpu):
    """The reference's executor loop (exec.py:392-453) replayed over the fixture through _C.launch_by_id."""
    import oracle
    init = _fixture_inputs()
    env = {v["vid"]: (Tensor.from_numpy(init[v["vid"]]) if v["vid"] in init else Tensor.zeros(v["shape"], "f16"))
           for v in FIX["values"]}
    _C.trace_reset()
    _C.trace_enable(True)
    for it in FIX["lowered"]:
        schema, payload = pack_attrs(it["op"], it["attrs"])
        _C.launch_by_id(it["kernel_id"], OpKind(OPNAME_TO_KIND[it["op"]]), [env[i] for i in it["inputs"]],
                        [env[o] for o in it["outputs"]], schema, payload, 0)
    _C.device_sync()
    assert _C.trace_get() == FIX["runtime_trace"]

    ref_env = {v["vid"]: (init[v["vid"]].astype(np.float32) if v["vid"] in init else np.zeros(v["shape"], np.float32))
               for v in FIX["values"]}
    oracle.run_lowered(FIX["lowered"], ref_env, {v["vid"]: "f16" for v in FIX["values"]}, np.float64)
    for v in FIX["values"]:
        got = env[v["vid"]].float_numpy()
        assert np.allclose(got, ref_env[v["vid"]], rtol=4e-3, atol=2e-3), v["name"]


@pytest.mark.gpu
def test_fixture_graph_as_a_captured_plan(gpu):
    import oracle
    init = _fixture_inputs()
    vals = [ValueSpec(v["vid"], v["name"], tuple(v["shape"]), _TORCH_DT[v["dtype"]], persistent=True) for v in FIX["values"]]
    plan = Plan("fixture", vals, FIX["lowered"])
    assert plan.kernel_ids() == [it["kernel_id"] for it in FIX["lowered"]]
    for vid, arr in init.items():
        plan.tensor(vid).copy_from_host(arr)
    plan.capture()
    plan.replay(3)
    plan.sync()
    ref_env = {v["vid"]: (init[v["vid"]].astype(np.float32) if v["vid"] in init else np.zeros(v["shape"], np.float32))
               for v in FIX["values"]}
    for _ in range(3):
        oracle.run_lowered(FIX["lowered"], ref_env, {v["vid"]: "f16" for v in FIX["values"]}, np.float64)
    for name in ("0.W", "0.b", "2.W", "2.b"):
        vid = plan.vid(name)
        assert np.allclose(plan.tensor(vid).float_numpy(), ref_env[vid], rtol=4e-3, atol=2e-3), name
    plan.close()
