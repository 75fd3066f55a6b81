"""The tracing front end and its lowering stages against the reference's committed end-to-end dumps.

The fixture (tests/golden/boundary_fixture.json) is the output of the reference's
python_framework_test/v2_kid_trace_by_id_test.py: a 2-layer f16 MLP, B=64, D=8, MSE + SGD(lr=0.01). The same
model traced through this front end must give the same IR, the same lowered list with the same kernel ids,
the same binding roles and byte-identical text dumps; on a GPU the executor must reproduce the runtime
trace and the oracle's numbers.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest

from aicf_cuda import core_v2 as cv

FIX = json.loads((Path(__file__).parent / "golden" / "boundary_fixture.json").read_text())
B, D, LR = 64, 8, 1e-2


def build_fixture_model(dtype="f16"):
    sx = cv.sym_tensor(name="x", shape=(B, D), dtype=dtype)
    st = cv.sym_tensor(name="t", shape=(B, D), dtype=dtype)
    sW0 = cv.sym_tensor(name="0.W", shape=(D, D), dtype=dtype)
    sb0 = cv.sym_tensor(name="0.b", shape=(D,), dtype=dtype)
    sW1 = cv.sym_tensor(name="2.W", shape=(D, D), dtype=dtype)
    sb1 = cv.sym_tensor(name="2.b", shape=(D,), dtype=dtype)
    lin0 = cv.linear(sx, sW0, sb0, name="lin0_out")
    r0 = cv.relu(lin0, name="relu0_out")
    r0s = cv.save(r0, name="relu0_saved")
    lin1 = cv.linear(r0, sW1, sb1, name="lin1_out")
    dY = cv.mse_grad(lin1, st, name="dY")
    d_r0, dW1, db1 = cv.linear_bwd(r0, sW1, dY, bias=True, dx_name="d_relu0_out", dW_name="d_2.W", db_name="d_2.b")
    d_lin0 = cv.relu_bwd(d_r0, r0s, name="d_lin0_out")
    _dx, dW0, db0 = cv.linear_bwd(sx, sW0, d_lin0, bias=True, dx_name="d_x", dW_name="d_0.W", db_name="d_0.b")
    cv.sgd_step(sW0, dW0, lr=LR)
    cv.sgd_step(sb0, db0, lr=LR)
    cv.sgd_step(sW1, dW1, lr=LR)
    cv.sgd_step(sb1, db1, lr=LR)


def traced():
    return cv.trace_ir(build_fixture_model, name="v2_kid_trace_by_id_test")


def test_trace_gives_the_reference_ir():
    ir = traced()
    assert [(v.id, v.name, list(v.shape), v.dtype.split(".")[-1]) for _, v in sorted(ir.values.items())] == \
        [(v["vid"], v["name"], v["shape"], v["dtype"]) for v in FIX["values"]]
    assert [{"op": n.op, "inputs": n.inputs, "outputs": n.outputs, "attrs": n.attrs} for n in ir.nodes] == FIX["ir_nodes"]
    assert cv.dump_ir(ir) == FIX["text"]["ir"]


def test_stages_give_the_reference_lowered_list_with_kernel_ids():
    ir = traced()
    stage_a = cv.lower_to_backend_ops(ir)
    assert [it["op"] for it in stage_a] == [
        "gemm", "bias_add", "relu", "copy_saved", "gemm", "bias_add", "mse_grad", "gemm", "gemm", "reduce_sum", "relu_bwd",
        "gemm", "gemm", "reduce_sum", "sgd_step", "sgd_step", "sgd_step", "sgd_step"]
    assert all("kernel_id" not in it for it in stage_a)
    stage_b = cv.apply_kernel_decisions_stageB(ir, stage_a)
    assert [it.get("kernel_id") for it in stage_b if it["op"] == "gemm"] == [None] * 6      # stage B only upgrades
    stage_c = cv.stageC_fuse_gemm_epilogue(ir, stage_b)
    lowered = cv.apply_kernel_selection(ir, stage_c, overwrite=False)
    assert lowered == FIX["lowered"]
    assert cv.compile_lowered(ir) == FIX["lowered"]
    assert cv.dump_lowered(lowered, name="v2_kid_trace_by_id_test") == FIX["text"]["lowered"]


def test_binding_plan_roles_and_dump():
    ir = traced()
    plan = cv.build_binding_plan(ir)
    assert {s.vid: s.role for s in plan.specs.values()} == {v["vid"]: v["role"] for v in FIX["values"]}
    assert cv.dump_plan(plan, name="v2_kid_trace_by_id_test") == FIX["text"]["plan"]
    # the input names win over the static prefixes, the static prefixes over the parameter pattern
    ir2 = cv.IRGraph("roles")
    for nm in ("x", "d_0.W", "opt.m.0.W", "3.W", "3.w", "grad_x"):
        ir2.new_value(name=nm, shape=(2,), dtype="f32")
    roles = [s.role for _, s in sorted(cv.build_binding_plan(ir2, opts=cv.PlanOptions(input_names={"x", "d_0.W"})).specs.items())]
    assert roles == ["input", "input", "static", "param", "static", "static"]


def test_kernel_selection_by_dtype_and_shape():
    ir = cv.IRGraph("sel")
    h = ir.new_value(name="h", shape=(4, 7), dtype="f16")       # odd last dim, even count
    f = ir.new_value(name="f", shape=(4, 8), dtype="f32")
    o = ir.new_value(name="o", shape=(3, 3), dtype="f16")       # odd count
    bf = ir.new_value(name="bf", shape=(4, 8), dtype="bf16")
    s32 = ir.new_value(name="s", shape=(7,), dtype="f32")
    ops = [{"op": "relu", "inputs": [h.id], "outputs": [h.id], "attrs": {}},
           {"op": "relu", "inputs": [f.id], "outputs": [f.id], "attrs": {}},
           {"op": "sgd_step", "inputs": [h.id, h.id], "outputs": [h.id], "attrs": {"lr": 0.1}},
           {"op": "sgd_step", "inputs": [o.id, o.id], "outputs": [o.id], "attrs": {"lr": 0.1}},
           {"op": "reduce_sum", "inputs": [h.id], "outputs": [s32.id], "attrs": {"axis": 0}},
           {"op": "gemm", "inputs": [bf.id, bf.id], "outputs": [bf.id], "attrs": {}},
           {"op": "adam_step", "inputs": [f.id] * 6, "outputs": [f.id] * 3, "attrs": {}}]
    out = cv.apply_kernel_selection(ir, cv.apply_kernel_decisions_stageB(ir, ops), overwrite=False)
    assert [it.get("kernel_id") for it in out] == [
        "relu_f16_v0", "relu_f32_v0", "sgd_step_f16_half2_v0", "sgd_step_f16_v0", "reduce_sum_keep_lastdim_f16_to_f32_v0",
        None, "adam_step_f32_v0"]


def test_fusion_rules():
    g = {"op": "gemm", "inputs": [0, 1], "outputs": [2], "attrs": {"transB": True}}
    bias = {"op": "bias_add", "inputs": [2, 3], "outputs": [2], "attrs": {}}
    act = {"op": "relu", "inputs": [2], "outputs": [4], "attrs": {}}
    assert cv.stageC_fuse_gemm_epilogue(None, [g, bias, act]) == [
        {"op": "gemm_epilogue", "inputs": [0, 1, 3], "outputs": [4],
         "attrs": {"transB": True, "epilogue_act": "relu", "epilogue_bias": True}}]
    assert cv.stageC_fuse_gemm_epilogue(None, [g, act]) == [
        {"op": "gemm_epilogue", "inputs": [0, 1], "outputs": [4],
         "attrs": {"transB": True, "epilogue_act": "relu", "epilogue_bias": False}}]
    assert cv.apply_opt_rules(None, [g, bias, act]) == [
        {"op": "gemm_epilogue", "inputs": [0, 1, 3], "outputs": [4], "attrs": {"transB": True, "epilogue": "bias_relu"}}]
    assert [it["op"] for it in cv.apply_opt_rules(None, [g, act])] == ["gemm", "relu"]          # bias is mandatory there
    # not fused: bias_add out of place, relu reading another value, or an op in between
    oop = dict(bias, outputs=[5])
    assert [it["op"] for it in cv.stageC_fuse_gemm_epilogue(None, [g, oop, act])] == ["gemm", "bias_add", "relu"]
    other = dict(act, inputs=[7])
    assert [it["op"] for it in cv.stageC_fuse_gemm_epilogue(None, [g, bias, other])] == ["gemm", "bias_add", "relu"]
    cp = {"op": "copy", "inputs": [2], "outputs": [6], "attrs": {}}
    assert [it["op"] for it in cv.stageC_fuse_gemm_epilogue(None, [g, bias, cp, act])] == ["gemm", "bias_add", "copy", "relu"]


def test_saved_activation_copies_can_be_elided():
    low = cv.elide_saved_copies(None, FIX["lowered"])
    assert len(low) == len(FIX["lowered"]) - 1 and all(it["op"] != "copy_saved" for it in low)
    relu_bwd = [it for it in low if it["op"] == "relu_bwd"][0]
    assert relu_bwd["inputs"] == [11, 4]                                   # reads relu0_out itself, not its copy
    assert FIX["lowered"][8]["inputs"] == [11, 5]                          # the input list was not modified
    # a source that is overwritten before the saved value is read keeps its copy
    ops = [{"op": "copy_saved", "inputs": [1], "outputs": [2], "attrs": {}},
           {"op": "relu", "inputs": [1], "outputs": [1], "attrs": {}},
           {"op": "relu_bwd", "inputs": [3, 2], "outputs": [4], "attrs": {}}]
    assert cv.elide_saved_copies(None, ops) == ops
    # ... while one that is overwritten only after the last read does not
    ops2 = [ops[0], ops[2], ops[1]]
    assert [it["op"] for it in cv.elide_saved_copies(None, ops2)] == ["relu_bwd", "relu"]


def test_tracing_rules_and_errors():
    with pytest.raises(RuntimeError, match="tracing-only"):
        cv.relu(cv.sym_tensor(name="x", shape=(2, 2), dtype="f32"))
    with pytest.raises(RuntimeError, match="not tracing"):
        cv.get_ir()

    def bad_linear():
        cv.linear(cv.sym_tensor(name="x", shape=(2, 3), dtype="f32"), cv.sym_tensor(name="0.W", shape=(4, 5), dtype="f32"))
    with pytest.raises(RuntimeError, match="shape mismatch"):
        cv.trace_ir(bad_linear)
    assert not cv.is_tracing()                                           # the state is restored after an error

    def adam():
        p, g = (cv.sym_tensor(name=n, shape=(4,), dtype="f32") for n in ("0.W", "d_0.W"))
        m, v = (cv.sym_tensor(name=n, shape=(4,), dtype="f32") for n in ("opt.m.0.W", "opt.v.0.W"))
        step = cv.sym_tensor(name="opt.step", shape=(), dtype="i32")
        b1, b2 = (cv.sym_tensor(name=n, shape=(), dtype="f32") for n in ("opt.bc1_inv", "opt.bc2_inv"))
        step2 = cv.step_inc(step, name="opt.step")
        o1, o2 = cv.bias_corr(step2, b1, b2, beta1=0.9, beta2=0.999)
        cv.adam_step(p, g, m, v, o1, o2, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
        with pytest.raises(RuntimeError, match="int32/int64"):
            cv.step_inc(p)
    ir = cv.trace_ir(adam, name="adam")
    assert [n.op for n in ir.nodes] == ["StepInc", "BiasCorr", "AdamStep"]
    low = cv.compile_lowered(ir)
    assert [(it["op"], it["kernel_id"]) for it in low] == [("step_inc", "step_inc_v0"), ("bias_corr", "bias_corr_v0"),
                                                            ("adam_step", "adam_step_f32_v0")]
    assert low[2]["inputs"][0] == low[2]["outputs"][0] and low[2]["outputs"] == [low[2]["inputs"][i] for i in (0, 2, 3)]
    assert low[2]["attrs"] == {"lr": 1e-3, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8}
    with pytest.raises(RuntimeError, match="unsupported IR op"):
        bad = cv.IRGraph("bad")
        bad.emit(op="Conv2d", inputs=[], outputs=[])
        cv.lower_to_backend_ops(bad)
    # nested tracing restores the outer graph
    outer = cv.IRGraph("outer")
    with cv.tracing(outer):
        cv.trace_ir(lambda: None, name="inner")
        assert cv.get_ir() is outer


def test_dtype_spellings():
    torch = pytest.importorskip("torch")
    for given, short in ((torch.float16, "f16"), (torch.bfloat16, "bf16"), (torch.float32, "f32"), (np.float16, "f16"),
                         (np.dtype("float32"), "f32"), ("torch.int32", "i32"), ("float16", "f16"), ("bf16", "bf16")):
        assert cv.short_dtype(given) == short
    assert cv.long_dtype("f16") == str(torch.float16)
    with pytest.raises(ValueError):
        cv.short_dtype("complex64")


# ---- GPU ---------------------------------------------------------------------------------------------------
def _host_inputs(seed=0):
    rng = np.random.default_rng(seed)
    h = lambda *s: rng.standard_normal(s).astype(np.float16)
    return {"x": h(B, D), "t": h(B, D)}, {"0.W": h(D, D), "0.b": h(D), "2.W": h(D, D), "2.b": h(D)}


@pytest.mark.gpu
def test_executor_runs_the_fixture_model_like_the_reference(gpu):
    from aicf_cuda import Tensor
    import oracle
    ir = traced()
    lowered = cv.compile_lowered(ir)
    ex = cv.PlannedExecutor(ir=ir, lowered=lowered, plan=cv.build_binding_plan(ir), opts=cv.ExecOptions(require_kernel_id=True))
    h_in, h_par = _host_inputs()
    inputs = {k: Tensor.from_numpy(v) for k, v in h_in.items()}
    params = {k: Tensor.from_numpy(v) for k, v in h_par.items()}
    ex.trace_reset()
    ex.trace_enable(True)
    env = ex.run(inputs=inputs, params=params, reuse_static=True)
    ex.sync()
    assert ex.trace_get() == FIX["runtime_trace"]
    names = {v.id: v.name for v in ir.values.values()}
    by_name = {**h_in, **h_par}
    ref = {vid: (by_name[nm].astype(np.float32) if nm in by_name else np.zeros(ir.values[vid].shape, np.float32))
           for vid, nm in names.items()}
    oracle.run_lowered(lowered, ref, {vid: "f16" for vid in names}, np.float64)
    for vid, name in names.items():
        if name == "lin0_out":
            continue                                                     # fused away: never written
        np.testing.assert_allclose(env[vid].float_numpy(), ref[vid], rtol=4e-3, atol=2e-3, err_msg=name)
    # parameters were updated in place, in the caller's tensors
    assert not np.array_equal(params["0.W"].numpy(), h_par["0.W"])


@pytest.mark.gpu
def test_executor_with_elided_copies_gives_the_same_parameters(gpu):
    from aicf_cuda import Tensor
    ir = traced()
    h_in, h_par = _host_inputs(2)
    results = []
    for lowered in (cv.compile_lowered(ir), cv.elide_saved_copies(ir, cv.compile_lowered(ir))):
        ex = cv.PlannedExecutor(ir=ir, lowered=lowered, plan=cv.build_binding_plan(ir))
        params = {k: Tensor.from_numpy(v) for k, v in h_par.items()}
        for _ in range(2):
            ex.run(inputs={k: Tensor.from_numpy(v) for k, v in h_in.items()}, params=params, reuse_static=False)
        ex.sync()
        results.append({k: v.numpy() for k, v in params.items()})
    for k in results[0]:
        np.testing.assert_array_equal(results[0][k], results[1][k], err_msg=k)


@pytest.mark.gpu
def test_executor_capture_replay_equals_repeated_runs(gpu):
    from aicf_cuda import Tensor
    ir = traced()
    lowered = cv.compile_lowered(ir)
    h_in, h_par = _host_inputs(1)
    results = []
    for mode in ("run", "replay"):
        ex = cv.PlannedExecutor(ir=ir, lowered=lowered, plan=cv.build_binding_plan(ir))
        inputs = {k: Tensor.from_numpy(v) for k, v in h_in.items()}
        params = {k: Tensor.from_numpy(v) for k, v in h_par.items()}
        if mode == "run":
            for _ in range(3):
                ex.run(inputs=inputs, params=params)
        else:
            with pytest.raises(RuntimeError, match="before capture"):
                ex.replay(1)
            ex.capture(inputs=inputs, params=params)
            ex.replay(3)
        ex.sync()
        from aicf_cuda import _C
        _C.device_sync()
        results.append({k: v.numpy() for k, v in params.items()})
        ex.reset_graph()
    for k in results[0]:
        np.testing.assert_array_equal(results[0][k], results[1][k], err_msg=k)
    ex2 = cv.PlannedExecutor(ir=ir, lowered=lowered, plan=cv.build_binding_plan(ir))
    with pytest.raises(KeyError, match="unknown or ambiguous"):
        ex2.run(inputs={"nope": Tensor.from_numpy(h_in["x"])}, params={})
    with pytest.raises(RuntimeError, match="shape mismatch"):
        ex2.run(inputs={"x": Tensor.from_numpy(h_in["x"][:8]), "t": Tensor.from_numpy(h_in["t"])},
                params={k: Tensor.from_numpy(v) for k, v in h_par.items()})
    with pytest.raises(RuntimeError, match="env missing"):
        ex2.run(inputs={"x": Tensor.from_numpy(h_in["x"])}, params={})
    no_ids = [{k: v for k, v in it.items() if k != "kernel_id"} for it in lowered]
    with pytest.raises(RuntimeError, match="require_kernel_id"):
        cv.PlannedExecutor(ir=ir, lowered=no_ids, plan=cv.build_binding_plan(ir), opts=cv.ExecOptions(require_kernel_id=True))


# ---- differential goldens: the same models traced by the reference's own front end -----------------------------
GOLD = json.loads((Path(__file__).parent / "golden" / "frontend_golden.json").read_text())


def _models():
    from frontend_models import MODELS
    return MODELS


@pytest.mark.parametrize("spec", _models(), ids=lambda s: s["name"])
def test_every_stage_equals_the_reference_front_end(spec):
    from frontend_models import build_model
    g = GOLD[spec["name"]]
    ir = cv.trace_ir(lambda: build_model(cv, spec, spec["dtype"], "f32", "i32"), name=spec["name"])
    assert cv.dump_ir(ir) == g["ir_text"]
    a = cv.lower_to_backend_ops(ir)
    assert a == g["stage_a"]
    b = cv.apply_kernel_decisions_stageB(ir, a)
    assert b == g["stage_b"]
    c = cv.stageC_fuse_gemm_epilogue(ir, b)
    assert c == g["stage_c"]
    final = cv.apply_kernel_selection(ir, c, overwrite=False)
    assert final == g["final"] == cv.compile_lowered(ir)
    assert cv.apply_kernel_selection(ir, cv.apply_opt_rules(ir, a)) == g["opt_rules_then_select"]
    assert cv.dump_plan(cv.build_binding_plan(ir), name=spec["name"]) == g["plan_text"]
    assert cv.dump_lowered(final, name=spec["name"]) == g["final_text"]


def test_temporaries_freed_mid_trace_do_not_alias_values():
    """Values are keyed by object identity and the object is held for the length of the trace, so a model written with
    rebinding locals (h = relu(h)) traces the same graph as one that keeps every tensor alive."""
    from frontend_models import MODELS, build_model
    spec = MODELS[1]
    ir = cv.trace_ir(lambda: build_model(cv, spec, spec["dtype"], "f32", "i32", keep_alive=False), name=spec["name"])
    assert cv.dump_ir(ir) == GOLD[spec["name"]]["ir_text"]


def test_reference_import_paths_resolve_to_this_front_end():
    import aicf_fw.core_v2 as pkg
    from aicf_fw.core_v2 import PlannedExecutor, trace_ir  # noqa: F401
    from aicf_fw.core_v2.exec import ExecOptions  # noqa: F401
    from aicf_fw.core_v2.lower import lower_to_backend_ops
    from aicf_fw.core_v2.ops import linear_bwd, relu_bwd, save, sgd_step  # noqa: F401
    from aicf_fw.core_v2.plan import apply_kernel_decisions_stageB, build_binding_plan  # noqa: F401
    from aicf_fw.core_v2.rewrites.stageC_fuse_epilogue import stageC_fuse_gemm_epilogue
    assert pkg.trace_ir is cv.trace_ir and lower_to_backend_ops is cv.lower_to_backend_ops
    assert stageC_fuse_gemm_epilogue is cv.stageC_fuse_gemm_epilogue
    assert set(pkg.__all__) >= {"trace_ir", "dump_ir", "dump_lowered", "dump_plan", "lower_to_backend_ops", "build_binding_plan",
                                "BindingPlan", "PlanOptions", "SymTensor", "sym_tensor", "linear", "relu", "mse_grad",
                                "PlannedExecutor", "ExecOptions"}


# ---- compile_train_step -----------------------------------------------------------------------------------
def test_compile_train_step_graph_shape():
    """Host-side part: the traced and lowered step (no device needed until the first run)."""
    from aicf_cuda.train_step import same_name_is_same_storage
    ir = cv.IRGraph("alias")
    a = ir.new_value(name="opt.step", shape=(), dtype="i32")
    b = ir.new_value(name="opt.step", shape=(), dtype="i32")
    c = ir.new_value(name="x", shape=(2,), dtype="f32")
    d = ir.new_value(name="x", shape=(2,), dtype="f32")
    low = [{"op": "step_inc", "inputs": [a.id], "outputs": [b.id], "attrs": {}},
           {"op": "copy", "inputs": [c.id], "outputs": [d.id], "attrs": {}}]
    out = same_name_is_same_storage(ir, low)
    assert out[0]["inputs"] == out[0]["outputs"] == [a.id]               # optimizer state: one buffer per name
    assert out[1]["inputs"] == [c.id] and out[1]["outputs"] == [d.id]     # other names are left alone


@pytest.mark.gpu
@pytest.mark.parametrize("optimizer,dtype", [("adam", "f32"), ("sgd", "f16"), ("sgd", "f32")])
def test_compile_train_step_matches_the_oracle_eager_and_replayed(gpu, optimizer, dtype):
    import oracle
    from aicf_cuda.train_step import compile_train_step
    dims, Bn, steps = [24, 32, 16, 8], 48, 4
    rng = np.random.default_rng(3)
    x = rng.standard_normal((Bn, dims[0])).astype(np.float32)
    t = rng.standard_normal((Bn, dims[-1])).astype(np.float32)
    init = {}
    for i in range(len(dims) - 1):
        init[f"{2 * i}.W"] = (rng.standard_normal((dims[i + 1], dims[i])) * 0.2).astype(np.float32)
        init[f"{2 * i}.b"] = (rng.standard_normal((dims[i + 1],)) * 0.1).astype(np.float32)
    kw = dict(B=Bn, dtype=dtype, optimizer=optimizer, lr=0.01, loss_scale=2.0 / (Bn * dims[-1]), params=init)

    eager = compile_train_step(dims, **kw)
    for _ in range(steps):
        eager.train_step({"x": x, "t": t})
    eager.sync()
    graphed = compile_train_step(dims, **kw)
    graphed.capture({"x": x, "t": t})
    graphed.replay(steps, sync=True)
    graphed.sync()

    # oracle: the same lowered list interpreted on the host
    ir, lowered = eager.ir, eager.lowered
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == "f16" else (lambda a: a)
    dts = {vid: cv.short_dtype(v.dtype) for vid, v in ir.values.items()}
    env = {vid: np.zeros(v.shape, np.int32 if dts[vid] == "i32" else np.float32) for vid, v in ir.values.items()}
    by_name = {v.name: vid for vid, v in sorted(ir.values.items(), reverse=True)}
    for nm, a in {**init, "x": x, "t": t}.items():
        env[by_name[nm]] = rnd(a.copy())
    f32 = lambda it: dict(it, attrs={k: (float(np.float32(v)) if isinstance(v, float) else v) for k, v in it["attrs"].items()})
    for _ in range(steps):
        oracle.run_lowered([f32(it) for it in lowered], env, dts, np.float64)
    tol = dict(rtol=2e-2, atol=2e-3) if dtype == "f16" else dict(rtol=2e-4, atol=2e-5)
    for nm in init:
        want = env[by_name[nm]]
        bad = ~np.isclose(eager.params[nm].float_numpy(), want, **tol)
        # Adam divides by sqrt(v): where a gradient is within rounding of zero the fp32 and fp64 updates differ by up
        # to lr, so a small fraction of elements may sit outside the tolerance; SGD must match everywhere.
        assert bad.mean() <= (0.01 if optimizer == "adam" else 0.0), f"eager {nm}: {bad.sum()} of {bad.size} differ"
        np.testing.assert_array_equal(graphed.params[nm].numpy(), eager.params[nm].numpy(), err_msg=f"replay {nm}")
    if optimizer == "adam":
        assert int(eager.value("opt.step").numpy()) == steps == int(graphed.value("opt.step").numpy())


@pytest.mark.gpu
def test_front_end_and_executor_take_torch_dtypes_and_tensors(gpu):
    """What a script written against the reference does: torch dtypes and devices in sym_tensor, torch CUDA tensors
    into PlannedExecutor.run. torch is only duck-typed (data_ptr / shape / dtype / is_contiguous)."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("torch sees no CUDA device")
    from aicf_fw.core_v2 import PlannedExecutor, dump_lowered, trace_ir
    from aicf_fw.core_v2.exec import ExecOptions
    from aicf_fw.core_v2.lower import lower_to_backend_ops
    from aicf_fw.core_v2.ops import linear, linear_bwd, mse_grad, relu, relu_bwd, save, sgd_step, sym_tensor
    from aicf_fw.core_v2.plan import apply_kernel_decisions_stageB, build_binding_plan
    from aicf_fw.core_v2.rewrites.stageC_fuse_epilogue import stageC_fuse_gemm_epilogue
    from aicf_fw.core_v2.kernel_select import apply_kernel_selection
    device, dtype = torch.device("cuda:0"), torch.float16

    def build():
        sx, st = (sym_tensor(name=n, shape=(B, D), dtype=dtype, device=device) for n in ("x", "t"))
        sW0, sW1 = (sym_tensor(name=n, shape=(D, D), dtype=dtype, device=device) for n in ("0.W", "2.W"))
        sb0, sb1 = (sym_tensor(name=n, shape=(D,), dtype=dtype, device=device) for n in ("0.b", "2.b"))
        r0 = relu(linear(sx, sW0, sb0, name="lin0_out"), name="relu0_out")
        r0s = save(r0, name="relu0_saved")
        dY = mse_grad(linear(r0, sW1, sb1, name="lin1_out"), st, name="dY")
        d_r0, dW1, db1 = linear_bwd(r0, sW1, dY, bias=True, dx_name="d_relu0_out", dW_name="d_2.W", db_name="d_2.b")
        _dx, dW0, db0 = linear_bwd(sx, sW0, relu_bwd(d_r0, r0s, name="d_lin0_out"), bias=True, dx_name="d_x",
                                   dW_name="d_0.W", db_name="d_0.b")
        for p, g in ((sW0, dW0), (sb0, db0), (sW1, dW1), (sb1, db1)):
            sgd_step(p, g, lr=LR)

    ir = trace_ir(build, name="v2_kid_trace_by_id_test")
    lowered = apply_kernel_selection(ir, stageC_fuse_gemm_epilogue(ir, apply_kernel_decisions_stageB(ir, lower_to_backend_ops(ir))),
                                     overwrite=False)
    assert dump_lowered(lowered, name="v2_kid_trace_by_id_test") == FIX["text"]["lowered"]
    h_in, h_par = _host_inputs(5)
    t_in = {k: torch.from_numpy(v).to(device) for k, v in h_in.items()}
    t_par = {k: torch.from_numpy(v).to(device) for k, v in h_par.items()}
    ex = PlannedExecutor(ir=ir, lowered=lowered, plan=build_binding_plan(ir), opts=ExecOptions(require_kernel_id=True))
    ex.trace_reset()
    ex.trace_enable(True)
    ex.run(inputs=t_in, params=t_par, reuse_static=True)
    torch.cuda.synchronize()
    assert ex.trace_get() == FIX["runtime_trace"]
    # the same step on aicf_cuda.Tensor buffers gives the same parameters, bit for bit
    from aicf_cuda import Tensor
    ex2 = cv.PlannedExecutor(ir=ir, lowered=lowered, plan=cv.build_binding_plan(ir))
    a_par = {k: Tensor.from_numpy(v) for k, v in h_par.items()}
    ex2.run(inputs={k: Tensor.from_numpy(v) for k, v in h_in.items()}, params=a_par)
    ex2.sync()
    for k in h_par:
        np.testing.assert_array_equal(t_par[k].cpu().numpy(), a_par[k].numpy(), err_msg=k)
        assert not np.array_equal(t_par[k].cpu().numpy(), h_par[k]), f"{k} was not updated in place"


# ---- AICF_WARMUP: a step that leaves the model where it is (reference exec.py:396,422-431) ---------------------------
def test_warmup_rewrites_step_inc_and_adam_lr():
    low = [{"op": "step_inc", "inputs": [0], "outputs": [1], "attrs": {}, "kernel_id": "step_inc_v0"},
           {"op": "step_inc", "inputs": [2], "outputs": [2], "attrs": {}, "kernel_id": "step_inc_v0"},
           {"op": "adam_step", "inputs": [3, 4, 5, 6, 7, 8], "outputs": [3, 5, 6], "attrs": {"lr": 0.01, "beta1": 0.9},
            "kernel_id": "adam_step_f32_v0"},
           {"op": "gemm", "inputs": [9, 10], "outputs": [11], "attrs": {"transB": True}, "kernel_id": "gemm_f32_naive_v0"}]
    ir = cv.IRGraph(name="w")
    ex = cv.PlannedExecutor(ir=ir, lowered=low, plan=cv.BindingPlan(name="w", inputs=[], params=[], statics=[], specs={}))
    assert ex._effective_lowered(False) == low
    w = ex._effective_lowered(True)
    assert [it["op"] for it in w] == ["copy", "adam_step", "gemm"]  # the in-place step_inc has nothing to copy
    assert (w[0]["inputs"], w[0]["outputs"], w[0]["kernel_id"]) == ([0], [1], "copy_i32_v0")
    assert w[1]["attrs"] == {"lr": 0.0, "beta1": 0.9} and low[2]["attrs"]["lr"] == 0.01  # the original list is untouched
    assert w[2] == low[3]


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["run", "replay"])
def test_warmup_mode_computes_gradients_and_moves_nothing(gpu, monkeypatch, mode):
    from aicf_cuda.train_step import compile_train_step
    dims, Bn = [24, 32, 8], 16
    rng = np.random.default_rng(5)
    batch = {"x": rng.standard_normal((Bn, dims[0])).astype(np.float32), "t": rng.standard_normal((Bn, dims[-1])).astype(np.float32)}

    def one_step(warm):
        if warm:
            monkeypatch.setenv("AICF_WARMUP", "1")
        else:
            monkeypatch.delenv("AICF_WARMUP", raising=False)
        ts = compile_train_step(dims, B=Bn, dtype="f32", optimizer="adam", lr=0.01, seed=1)
        before = {k: v.numpy() for k, v in ts.params.items()}
        if mode == "run":
            ts.train_step(batch)
        else:
            ts.capture(batch)
            ts.replay(1)
        ts.sync()
        return ts, before

    warm, w_before = one_step(True)
    real, r_before = one_step(False)
    for k in w_before:
        np.testing.assert_array_equal(warm.params[k].numpy(), w_before[k], err_msg=f"{k} moved in warm-up mode")
        assert not np.array_equal(real.params[k].numpy(), r_before[k]), f"{k} did not move in a normal step"
        np.testing.assert_array_equal(warm.value(f"d_{k}").numpy(), real.value(f"d_{k}").numpy(), err_msg=f"gradient of {k}")
        assert np.abs(warm.value(f"opt.m.{k}").numpy()).max() > 0, "moments are still updated, as in the reference"
    assert int(warm.value("opt.step").numpy()) == 0 and int(real.value("opt.step").numpy()) == 1
