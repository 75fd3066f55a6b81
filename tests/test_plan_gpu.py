"""The captured plan: small-MLP train steps (BASELINE config 1) against the NumPy execution of the same
lowered-op list, eager vs captured replay, arena reuse, and the process-global graph API."""
import struct

import numpy as np
import pytest

import oracle
from aicf_cuda import _C, DoubleBufferedStep, Plan, Tensor, build_mlp_train_step, f32_to_bf16_bits
from aicf_cuda._C import OpKind
from util import gemm_tuning

pytestmark = pytest.mark.gpu


def host_bits(arr, dtype):
    """Host array in the device's storage format (bf16 travels as uint16 bit patterns)."""
    if dtype == "bf16":
        return f32_to_bf16_bits(np.asarray(arr, np.float32))
    return np.asarray(arr, {"f32": np.float32, "f16": np.float16, "i32": np.int32}[dtype])


def make_plan(batch, dims, dtype, seed=0, **kw):
    vals, low = build_mlp_train_step(batch, dims, compute_dtype=dtype, **kw)
    plan = Plan(f"mlp_{dtype}", vals, low)
    params = oracle.mlp_params(dims, seed)
    x, y = oracle.mlp_batch(batch, dims[0], dims[-1], seed)
    env, dtypes = {}, {}
    for v in vals:
        dtypes[v.vid] = v.dtype
        if v.name == "x":
            arr = x
        elif v.name == "labels":
            arr = y
        elif v.name in params:
            arr = params[v.name]
        elif v.name.endswith(".W.lp"):
            arr = oracle.cast(params[v.name[:-3]], v.dtype)
        else:
            arr = np.zeros(v.shape, np.int32 if v.dtype == "i32" else np.float32)
        env[v.vid] = np.array(arr, copy=True)
        if v.name in ("x", "labels") or v.name in params or v.name.endswith(".W.lp"):
            plan.tensor(v.vid).copy_from_host(host_bits(arr, v.dtype))
    return plan, vals, low, env, dtypes


def test_small_mlp_ten_eager_steps_match_the_oracle(gpu):
    plan, vals, low, env, dtypes = make_plan(64, [784, 256, 10], "f32", seed=0, with_argmax=True)
    by = plan.by_name
    for step in range(10):
        plan.run()
        plan.sync()
        oracle.run_lowered(low, env, dtypes, np.float64)
        assert plan.tensor("loss").numpy()[0] == pytest.approx(float(env[by["loss"]][0]), rel=1e-5), f"step {step}"
        assert np.array_equal(plan.tensor("argmax").numpy(), env[by["argmax"]]), "argmax is bit-exact"
    assert int(plan.tensor("opt.step").numpy()[0]) == 10
    for name in ("0.W", "0.b", "2.W", "2.b"):
        got, want = plan.tensor(name).numpy(), env[by[name]]
        assert np.allclose(got, want, rtol=1e-4, atol=2e-6), name  # ten chained Adam steps on 1e-5-accurate grads
    assert _C.gemm_status() == 0
    plan.close()


def test_capture_replay_equals_eager_bit_for_bit(gpu):
    a, *_ = make_plan(64, [784, 256, 10], "f32", seed=0)
    b, *_ = make_plan(64, [784, 256, 10], "f32", seed=0)
    for _ in range(5):
        a.run()
    a.sync()
    with pytest.raises(RuntimeError, match="replay called before capture"):
        b.replay(1)
    b.capture()
    assert b.graph_nodes >= len(b.lowered)
    b.replay(5)
    b.sync()
    for name in ("0.W", "2.W", "2.b", "opt.m.0.W", "loss"):
        assert np.array_equal(a.tensor(name).numpy(), b.tensor(name).numpy()), name
    assert int(b.tensor("opt.step").numpy()[0]) == 5  # the device counter advanced without host help
    b.reset_graph()
    with pytest.raises(RuntimeError, match="replay called before capture"):
        b.replay(1)
    a.close()
    b.close()


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_mixed_precision_mlp_tracks_the_oracle(gpu, dtype):
    """16-bit GEMMs over fp32 master weights. Gradients are compared after the FIRST step: Adam's early
    updates are sign-like (|update| ~ lr whatever the gradient's size), so two correct executions that
    differ in the last bit drift apart within a few steps - the fp32 and fp64 NumPy runs of this graph
    already differ by 10% in d_0.W after three steps. The loss, an average, stays comparable."""
    dims = [256, 512, 384, 64]
    plan, vals, low, env, dtypes = make_plan(512, dims, dtype, seed=4, lr=1e-3, weight_decay=0.01)
    by = plan.by_name
    plan.capture()
    for step in range(4):
        plan.replay(1)
        plan.sync()
        oracle.run_lowered(low, env, dtypes, np.float64)
        assert plan.tensor("loss").numpy()[0] == pytest.approx(float(env[by["loss"]][0]), rel=2e-3), f"step {step}"
        if step == 0:
            for name in ("d_0.W", "d_2.W", "d_4.W", "d_0.b", "d_4.b"):  # 16-bit GEMM tolerance: 2e-2 normwise
                got, want = plan.tensor(name).numpy(), env[by[name]]
                assert np.max(np.abs(got - want)) <= 2e-2 * np.max(np.abs(want)), name
            for name in ("opt.m.2.W", "opt.v.2.W"):
                got, want = plan.tensor(name).numpy(), env[by[name]]
                assert np.max(np.abs(got - want)) <= 2e-2 * np.max(np.abs(want)), name
            for name in ("0.W", "4.W"):  # first Adam update is lr*sign(g): where g is rounding noise the sign may differ
                got, want = plan.tensor(name).numpy(), env[by[name]]
                off = np.abs(got - want) > 1e-5 * np.abs(want) + 2e-6
                assert off.mean() <= 5e-2 and np.max(np.abs(got - want)) <= 2.1e-3, name
    lp = plan.tensor("2.W.lp").float_numpy()
    assert np.array_equal(lp, oracle.cast(plan.tensor("2.W").numpy(), dtype)), "working copy == rounded master weight"
    assert _C.gemm_status() == 0
    plan.close()


def test_double_buffered_pipeline_equals_sequential_steps(gpu):
    """Two plans over shared parameters, inputs copied in on a second stream: same bits as one plan fed by hand."""
    dims, batch = [128, 256, 32], 256
    vals, low = build_mlp_train_step(batch, dims, compute_dtype="bf16")
    params = oracle.mlp_params(dims, seed=1)
    batches = [oracle.mlp_batch(batch, dims[0], dims[-1], seed=s) for s in (10, 11)]

    def load(plan):
        for name, w in params.items():
            plan.tensor(name).copy_from_host(w)
            if name.endswith(".W"):
                plan.tensor(name + ".lp").copy_from_host(f32_to_bf16_bits(w))

    seq = Plan("seq", vals, low)
    load(seq)
    seq.capture()
    losses_seq = []
    for t in range(6):
        x, y = batches[t % 2]
        seq.tensor("x").copy_from_host(x)
        seq.tensor("labels").copy_from_host(y)
        seq.replay(1)
        seq.sync()
        losses_seq.append(float(seq.tensor("loss").numpy()[0]))

    dbl = DoubleBufferedStep("dbl", vals, low)
    load(dbl.a)
    dbl.capture()
    losses, prev = [], None
    for t in range(6):
        slot = dbl.submit(list(batches[t % 2]))
        if prev is not None:
            losses.append(float(dbl.result(prev)[0]))
        prev = slot
    losses.append(float(dbl.result(prev)[0]))
    dbl.sync()
    assert losses == losses_seq
    for name in ("0.W", "2.W", "2.b", "opt.m.0.W"):
        assert np.array_equal(dbl.a.tensor(name).numpy(), seq.tensor(name).numpy()), name
    assert dbl.b.tensor("0.W").ptr == dbl.a.tensor("0.W").ptr and dbl.b.tensor("x").ptr != dbl.a.tensor("x").ptr
    dbl.close()
    seq.close()


def test_state_dict_resumes_training_bit_for_bit(gpu, tmp_path):
    """Checkpoint after 3 steps, restore into a fresh plan built from the JSON form, continue: same bits as 6 straight steps."""
    from aicf_cuda import plan_from_json, plan_to_json
    a, vals, low, *_ = make_plan(64, [784, 256, 10], "bf16", seed=0)
    a.capture()
    a.replay(3)
    a.sync()
    np.savez(tmp_path / "ckpt.npz", **a.state_dict())
    (tmp_path / "plan.json").write_text(plan_to_json("mlp", vals, low))
    a.replay(3)
    a.sync()
    name, vals2, low2 = plan_from_json((tmp_path / "plan.json").read_text())
    b = Plan(name, vals2, low2)
    b.load_state_dict(dict(np.load(tmp_path / "ckpt.npz")))
    x, y = oracle.mlp_batch(64, 784, 10, 0)
    b.tensor("x").copy_from_host(x)
    b.tensor("labels").copy_from_host(y)
    b.capture()
    b.replay(3)
    b.sync()
    assert sorted(a.state_names()) == sorted(b.state_names()) and "opt.step" in a.state_names()
    for n in a.state_names():
        assert np.array_equal(a.tensor(n).numpy(), b.tensor(n).numpy()), n
    a.close()
    b.close()


def test_arena_reuses_dead_buffers(gpu):
    vals, low = build_mlp_train_step(1024, [512, 512, 512, 512, 64], compute_dtype="bf16")
    plan = Plan("arena", vals, low)
    assert 0 < plan.arena_bytes < plan.arena_bytes_no_reuse
    plan.run()
    plan.sync()
    # the layout dump: parameters and inputs own their buffers, intermediates sit inside the arena, and some of them
    # share bytes (their live ranges do not overlap)
    import json
    doc = json.loads(plan.to_json())
    mm = {m["name"]: m for m in doc["memory_map"]}
    assert doc["arena_bytes"] == plan.arena_bytes and doc["format"] == "aicf_b200.plan/1" and len(doc["lowered"]) == len(low)
    assert mm["0.W"]["arena_offset"] is None and mm["x"]["arena_offset"] is None
    inside = [m for m in doc["memory_map"] if m["arena_offset"] is not None]
    assert inside and all(m["arena_offset"] + m["bytes"] <= plan.arena_bytes and m["arena_offset"] % 256 == 0 for m in inside)
    spans = sorted((m["arena_offset"], m["arena_offset"] + m["bytes"]) for m in inside)
    assert any(a2 < b1 for (a1, b1), (a2, b2) in zip(spans, spans[1:])), "no two values share arena bytes"
    assert sum(m["bytes"] for m in inside) > max(b for _, b in spans), "pooled values must not fit side by side"
    plan.close()


def test_global_graph_api_like_the_reference_binding(gpu):
    """graph_begin / op loop on the returned stream / graph_end / graph_launch, and the semantics the
    reference's framework test relies on: scalars are read from device memory at replay time."""
    n = 4096
    p0 = np.ones(n, np.float32)
    P, G, M, V = Tensor.from_numpy(p0), Tensor.from_numpy(np.full(n, 0.5, np.float32)), Tensor.zeros((n,)), Tensor.zeros((n,))
    bc1, bc2 = Tensor.from_numpy(np.array(0.1, np.float32)), Tensor.from_numpy(np.array(0.001, np.float32))
    pay = struct.pack("<ffff", 1e-2, 0.9, 0.999, 1e-8)
    with pytest.raises(RuntimeError, match="graph_launch called but no captured graph exists"):
        _C.graph_reset()
        _C.graph_launch()
    _C.trace_enable(True)  # the binding's default; another test may have switched it off
    s = _C.graph_begin()
    assert s != 0 and _C.graph_stream() == s
    _C.launch_by_id("adam_step_f32_v0", OpKind.AdamStep, [P, G, M, V, bc1, bc2], [P, M, V], 0x4D414441, pay, s)
    _C.graph_end()
    assert _C.trace_get() == ["kid:adam_step_f32_v0 kind:adam_step"]  # graph_begin cleared the trace
    assert np.array_equal(P.numpy(), p0), "capture records, it does not execute"
    _C.graph_launch()
    _C.device_sync()
    d1 = p0 - P.numpy()
    assert (d1 > 0).all()
    before = P.numpy()
    bc1.copy_from_host(np.array(1.0, np.float32))  # a 10x larger divisor => a visibly smaller update
    _C.graph_launch()
    _C.device_sync()
    d2 = before - P.numpy()
    assert (d2 < 0.5 * d1).all()
    _C.graph_reset()
    with pytest.raises(RuntimeError, match="graph_end called but not capturing"):
        _C.graph_end()


def test_fp32_mlp_on_the_tensor_cores_tracks_the_exact_plan(gpu):
    """compute_dtype f32 with fp32_gemm='3xtf32': every GEMM of the step (forward with bias/ReLU, dW, dX with the ReLU
    mask) runs under the 3xTF32 ids, whose staging copies come out of the plan's one workspace buffer. The loss follows
    the exact-fp32 plan and the oracle to 1e-5 on the first step and to 2e-4 over five captured replays."""
    dims, batch = [784, 256, 128, 10], 192
    exact, vals, low, env, dtypes = make_plan(batch, dims, "f32", seed=2)
    fast, vals_f, low_f, _, _ = make_plan(batch, dims, "f32", seed=2, fp32_gemm="3xtf32")
    gemm_ids = {it["kernel_id"] for it in low_f if it["op"] in ("gemm", "gemm_epilogue", "gemm_relu_bwd")}
    assert gemm_ids == {"gemm_f32_3xtf32_v0", "gemm_bias_relu_f32_3xtf32_v0", "gemm_relu_bwd_f32_3xtf32_v0"}
    by = exact.by_name
    fast.capture()
    for step in range(5):
        exact.run()
        fast.replay(1)
        exact.sync()
        fast.sync()
        oracle.run_lowered(low, env, dtypes, np.float64)
        want = float(env[by["loss"]][0])
        assert exact.tensor("loss").numpy()[0] == pytest.approx(want, rel=1e-5), f"exact, step {step}"
        # the first step sees the same weights (error of the GEMM path only, measured 2e-6); afterwards the two
        # trajectories separate slowly through Adam (2e-5 by the fifth step)
        assert fast.tensor("loss").numpy()[0] == pytest.approx(want, rel=1e-5 if step == 0 else 2e-4), f"3xtf32, step {step}"
    # Adam divides by sqrt(v): where a gradient is within rounding of zero the two plans may step in different
    # directions, so the weights are compared by the fraction of elements that moved apart
    for name in ("0.W", "2.W", "4.W"):
        a, b = exact.tensor(name).numpy(), fast.tensor(name).numpy()
        assert (~np.isclose(a, b, rtol=1e-3, atol=2e-5)).mean() <= 0.01, name
    assert _C.gemm_status() == 0
    exact.close()
    fast.close()


def test_small_batch_plan_with_gemms_split_over_k(gpu):
    """A small batch against wide layers: the forward and dX GEMMs (M = 64, K = 4096) are split over K by the launcher,
    with the parts in the plan's one workspace buffer. The captured replay equals the eager run bit for bit, and both
    follow the oracle; with the split switched off the plan needs no GEMM workspace and gives the same loss to GEMM
    tolerance."""
    dims, batch = [4096, 4096, 16], 64
    def two_steps(mode):
        eager, vals, low, env, dtypes = make_plan(batch, dims, "bf16", seed=6, lr=1e-3)
        graphed, *_ = make_plan(batch, dims, "bf16", seed=6, lr=1e-3)
        by = eager.by_name
        graphed.capture()
        for step in range(2):
            eager.run()
            graphed.replay(1)
            eager.sync()
            graphed.sync()
            oracle.run_lowered(low, env, dtypes, np.float64)
            assert eager.tensor("loss").numpy()[0] == pytest.approx(float(env[by["loss"]][0]), rel=2e-3), (mode, step)
            assert eager.tensor("loss").numpy()[0] == graphed.tensor("loss").numpy()[0], (mode, step)
        for name in ("0.W", "2.W", "0.b"):
            assert np.array_equal(eager.tensor(name).numpy(), graphed.tensor(name).numpy()), (mode, name)
        loss = float(eager.tensor("loss").numpy()[0])
        assert _C.gemm_status() == 0
        eager.close()
        graphed.close()
        return loss

    results = {"split": two_steps("split")}
    with gemm_tuning(splitk="0"):
        results["unsplit"] = two_steps("unsplit")
    assert results["split"] == pytest.approx(results["unsplit"], rel=2e-3)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_one_launch_optimizer_equals_one_launch_per_tensor(gpu, dtype):
    """The plan's optimizer as a single multi-tensor Adam launch against the per-tensor form: same parameters, moments
    and working copies, bit for bit, eagerly and replayed; and fewer kernels in the captured graph."""
    dims, batch = [96, 160, 64, 24], 32
    fused, *_ = make_plan(batch, dims, dtype, seed=2, fuse_adam=True)
    split, *_ = make_plan(batch, dims, dtype, seed=2, fuse_adam=False)
    assert "adam_step_f32_multi_v1" in fused.kernel_ids() and "adam_step_f32_multi_v1" not in split.kernel_ids()
    for plan in (fused, split):
        plan.run()
        plan.capture()
        plan.replay(3)
        plan.sync()
    names = [f"{2 * i}.{p}" for i in range(len(dims) - 1) for p in ("W", "b")]
    names += ["opt.m." + n for n in names] + ["opt.v." + n for n in names[:len(names)]]
    if dtype != "f32":
        names += [f"{2 * i}.W.lp" for i in range(len(dims) - 1)]
    for n in names:
        assert np.array_equal(fused.tensor(n).numpy(), split.tensor(n).numpy()), n
    assert int(fused.tensor("opt.step").numpy()[0]) == 4
    assert fused.graph_kernel_nodes == split.graph_kernel_nodes - (2 * (len(dims) - 1) - 1)
    assert _C.wait_status() == 0
    fused.close()
    split.close()
