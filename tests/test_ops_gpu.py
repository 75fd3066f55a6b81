"""Parity of the streaming kernels with the NumPy oracle, through the binding (launch_by_id / op_call)
and therefore through the C ABI. Shapes follow the reference's probe scripts
(python/cuda_binding_test/v2_*_probe.py) plus odd sizes, unaligned views and sizes past the limits the
reference mishandles. Tolerances: fp32 elementwise / reduce / Adam 1e-5 relative; integers exact;
16-bit outputs one rounding step of the output type."""
import struct

import numpy as np
import pytest

import oracle
from aicf_cuda import _C, Tensor, f32_to_bf16_bits
from aicf_cuda._C import OpKind
from util import assert_close_f32, by_id, dev, host, op_call

pytestmark = pytest.mark.gpu

SHAPES = [(1024,), (64, 256), (8, 32, 128)]
F = np.float32  # hyper-parameters travel as float32 payloads; the oracle gets the same rounded values
ADAM = 0x4D414441
BCOR = 0x524F4342
RSUM = 0x5253554D
SMCE = 0x45434D53


def rnd(shape, seed=0, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def scalar(v, dtype="f32"):
    return Tensor.from_numpy(np.array(v, np.float32 if dtype == "f32" else np.int32))  # rank 0


# ------------------------------------------------------------------ Adam
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("inplace", [False, True])
def test_adam_v0_reference_contract(gpu, shape, inplace):
    p, g, m, v = rnd(shape, 1), rnd(shape, 2, 1e-2), rnd(shape, 3, 1e-2), np.abs(rnd(shape, 4, 1e-3))
    bc1, bc2 = 1 - 0.9 ** 3, 1 - 0.999 ** 3
    P, G, M, V = dev(p), dev(g), dev(m), dev(v)
    Po, Mo, Vo = (P, M, V) if inplace else (Tensor.empty(shape), Tensor.empty(shape), Tensor.empty(shape))
    by_id("adam_step_f32_v0", OpKind.AdamStep, [P, G, M, V, scalar(bc1), scalar(bc2)], [Po, Mo, Vo], ADAM,
          struct.pack("<ffff", 1e-3, 0.9, 0.999, 1e-8))
    wp, wm, wv = oracle.adam_step_v0(p, g, m, v, F(bc1), F(bc2), F(1e-3), F(0.9), F(0.999), F(1e-8))
    assert_close_f32(host(Po), wp, what="p")
    assert_close_f32(host(Mo), wm, atol=1e-8, what="m")  # m' cancels: atol = 1e-6 x the operand scale
    assert_close_f32(host(Vo), wv, atol=1e-12, what="v")
    if not inplace:
        assert np.array_equal(host(P), p)  # inputs untouched out of place


def test_adam_v0_rejects_what_the_reference_rejects(gpu):
    shape = (64, 256)
    P, G, M, V = (dev(rnd(shape, i)) for i in range(4))
    sc = [scalar(0.5), scalar(0.5)]
    pay = struct.pack("<ffff", 1e-3, 0.9, 0.999, 1e-8)
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # gradient aliases an output
        by_id("adam_step_f32_v0", OpKind.AdamStep, [P, G, M, V] + sc, [G, M, V], ADAM, pay)
    h = Tensor.from_numpy(rnd(shape).astype(np.float16))
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # f16 parameters
        by_id("adam_step_f32_v0", OpKind.AdamStep, [h, G, M, V] + sc, [h, M, V], ADAM, pay)
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # schema 'ADAM' is mandatory
        by_id("adam_step_f32_v0", OpKind.AdamStep, [P, G, M, V] + sc, [P, M, V], 0, b"")
    one = Tensor.from_numpy(np.array([0.5], np.float32))        # rank-1 scalar is not rank 0
    with pytest.raises(RuntimeError, match="InvalidArgument"):
        by_id("adam_step_f32_v0", OpKind.AdamStep, [P, G, M, V, one, one], [P, M, V], ADAM, pay)


# 4096 * 300 + 1001: past the size where whole 16 KiB chunks go through the bulk-copy kernel, with a ragged tail
@pytest.mark.parametrize("n", [1, 3, 1001, 4096, 1 << 20, 4096 * 300 + 1001, 1 << 22])
@pytest.mark.parametrize("wd,dec", [(0.0, 0), (0.01, 0), (0.01, 1)])
def test_adam_fused_step_counter_weight_decay_and_bf16_copy(gpu, n, wd, dec):
    p, g = oracle.adam_inputs(n, seed=3)
    m, v = rnd((n,), 5, 1e-3), np.abs(rnd((n,), 6, 1e-6))
    P, G, M, V = dev(p), dev(g), dev(m), dev(v)
    step = Tensor.from_numpy(np.array([7], np.int32))
    lp = Tensor.empty((n,), "bf16")
    pay = struct.pack("<fffffI", 3e-4, 0.9, 0.999, 1e-8, wd, dec)
    by_id("adam_step_f32_fused_v1", OpKind.AdamStep, [P, G, M, V, step], [P, M, V, lp], ADAM, pay)
    wp, wm, wv = oracle.adam_step_fused(p, g, m, v, 7, F(3e-4), F(0.9), F(0.999), F(1e-8), weight_decay=F(wd), decoupled=bool(dec))
    assert_close_f32(host(P), wp, what="p")
    assert_close_f32(host(M), wm, atol=1e-9, what="m")   # operands ~1e-3: atol = 1e-6 x scale
    assert_close_f32(host(V), wv, atol=1e-12, what="v")  # operands ~1e-6
    assert np.array_equal(lp.numpy(), f32_to_bf16_bits(P.numpy()))  # bf16 copy is the rounded new parameter


def test_adam_v0_large_out_of_place(gpu):
    n = 4096 * 320 + 8
    p, g, m, v = rnd((n,), 1), rnd((n,), 2, 1e-2), rnd((n,), 3, 1e-2), np.abs(rnd((n,), 4, 1e-3))
    bc1, bc2 = 1 - 0.9 ** 3, 1 - 0.999 ** 3
    P, G, M, V = dev(p), dev(g), dev(m), dev(v)
    Po, Mo, Vo = Tensor.zeros((n,)), Tensor.zeros((n,)), Tensor.zeros((n,))
    by_id("adam_step_f32_v0", OpKind.AdamStep, [P, G, M, V, scalar(bc1), scalar(bc2)], [Po, Mo, Vo], ADAM,
          struct.pack("<ffff", 1e-3, 0.9, 0.999, 1e-8))
    wp, wm, wv = oracle.adam_step_v0(p, g, m, v, F(bc1), F(bc2), F(1e-3), F(0.9), F(0.999), F(1e-8))
    assert_close_f32(host(Po), wp, what="p")
    assert_close_f32(host(Mo), wm, atol=1e-8, what="m")
    assert_close_f32(host(Vo), wv, atol=1e-9, what="v")
    assert np.array_equal(host(P), p), "inputs untouched out of place"
    assert _C.wait_status() == 0


def test_adam_fused_unaligned_views_take_the_scalar_path(gpu):
    n = 1000
    base = [Tensor.zeros((n + 1,)) for _ in range(4)]
    arrs = [rnd((n,), i, 1e-2) for i in range(4)]
    arrs[3] = np.abs(arrs[3])
    views = []
    for b, a in zip(base, arrs):
        t = Tensor((n,), "f32", ptr=b.ptr + 4)  # 4-byte offset: not 16-byte aligned
        t.copy_from_host(a)
        views.append(t)
    step = Tensor.from_numpy(np.array([1], np.int32))
    by_id("adam_step_f32_fused_v1", OpKind.AdamStep, views + [step], views[:1] + views[2:], ADAM,
          struct.pack("<ffff", 1e-3, 0.9, 0.999, 1e-8))
    wp, wm, wv = oracle.adam_step_fused(*arrs, 1, F(1e-3), F(0.9), F(0.999), F(1e-8))
    assert_close_f32(host(views[0]), wp)
    assert_close_f32(host(views[2]), wm, atol=1e-8)  # operands ~1e-2: atol = 1e-6 x scale


@pytest.mark.parametrize("t", [1, 10, 0])
@pytest.mark.parametrize("rank0", [True, False])
def test_bias_corr(gpu, t, rank0):
    mk = (lambda v, dt: scalar(v, dt)) if rank0 else (lambda v, dt: Tensor.from_numpy(np.array([v], np.float32 if dt == "f32" else np.int32)))
    S, O1, O2 = mk(t, "i32"), mk(0, "f32"), mk(0, "f32")
    by_id("bias_corr_v0", OpKind.BiasCorr, [S], [O1, O2], BCOR, struct.pack("<ff", 0.9, 0.999))
    w1, w2 = oracle.bias_corr(t)
    w1, w2 = oracle.bias_corr(t, F(0.9), F(0.999))
    assert host(O1).ravel()[0] == pytest.approx(w1, rel=1e-5)
    assert host(O2).ravel()[0] == pytest.approx(w2, rel=1e-4)  # fp32 powf: 1-0.999^t cancels four digits
    with pytest.raises(RuntimeError, match="InvalidArgument"):
        by_id("bias_corr_v0", OpKind.BiasCorr, [S], [O1, O2], 0, b"")
    with pytest.raises(RuntimeError, match="InvalidArgument"):
        by_id("bias_corr_v0", OpKind.BiasCorr, [O1], [O1, O2], BCOR, struct.pack("<ff", 0.9, 0.999))


@pytest.mark.parametrize("shape", [(), (1,), (1024,), (64, 256)])
def test_step_inc_increments_the_output_buffer(gpu, shape):
    s = np.arange(int(np.prod(shape)) if shape else 1, dtype=np.int32).reshape(shape)
    S = Tensor.from_numpy(s)
    by_id("step_inc_v0", OpKind.StepInc, [S], [S])
    assert np.array_equal(S.numpy(), s + 1)
    SO = Tensor.from_numpy(s + 100)  # out of place: the reference never reads the input
    by_id("step_inc_v0", OpKind.StepInc, [S], [SO])
    assert np.array_equal(SO.numpy(), s + 101)


# ------------------------------------------------------------------ elementwise
def _cases():
    for shape in SHAPES:
        yield shape, "f32"
    yield (7, 33, 127), "f16"
    yield (7, 33, 127), "bf16"
    yield (64, 256), "f16"
    yield (64, 256), "bf16"


def _round(a, dt):
    return {"f32": lambda x: x, "f16": oracle.f16_round, "bf16": oracle.bf16_round}[dt](np.asarray(a, np.float32))


def _tol(dt):
    return {"f32": dict(rtol=1e-6, atol=1e-9), "f16": dict(rtol=1e-3, atol=1e-6), "bf16": dict(rtol=8e-3, atol=1e-6)}[dt]


@pytest.mark.parametrize("shape,dt", list(_cases()))
def test_elementwise_family(gpu, shape, dt):
    x, y = _round(rnd(shape, 1), dt), _round(rnd(shape, 2), dt)
    X, Y = dev(x, dt), dev(y, dt)
    O = Tensor.empty(shape, dt)
    sfx = dt
    by_id(f"relu_{sfx}_v0", OpKind.EltwiseRelu, [X], [O])
    assert np.array_equal(host(O), oracle.relu(x, np.float32))
    by_id(f"relu_bwd_{sfx}_v0", OpKind.ReluBwd, [X, Y], [O])
    assert np.array_equal(host(O), oracle.relu_bwd(x, y, np.float32))
    by_id(f"add_{sfx}_v0", OpKind.EltwiseAdd, [X, Y], [O])
    assert np.allclose(host(O), oracle.add(x, y), **_tol(dt))
    by_id(f"copy_{sfx}_v0", OpKind.Copy, [X], [O])
    assert np.array_equal(host(O), x)
    by_id(f"mse_grad_{sfx}_v0", OpKind.MseGrad, [X, Y], [O])
    assert np.allclose(host(O), oracle.mse_grad(x, y), **_tol(dt))
    by_id(f"mse_grad_{sfx}_v0", OpKind.MseGrad, [X, Y], [O], 0x4745534D, struct.pack("<f", 0.25))
    assert np.allclose(host(O), oracle.mse_grad(x, y, 0.25), **_tol(dt))
    by_id(f"sgd_step_{sfx}_v0", OpKind.SgdStep, [X, Y], [O])
    assert np.allclose(host(O), oracle.sgd_step(x, y), **_tol(dt))
    by_id(f"sgd_step_{sfx}_v0", OpKind.SgdStep, [X, Y], [O], 0x53444753, struct.pack("<f", 0.01))
    assert np.allclose(host(O), oracle.sgd_step(x, y, 0.01), **_tol(dt))
    by_id("grad_zero_v0", OpKind.GradZero, [O], [O])
    assert not host(O).any()
    if len(shape) >= 2:
        b = _round(rnd((shape[-1],), 3), dt)
        by_id(f"bias_add_{sfx}_v0", OpKind.BiasAdd, [X, dev(b, dt)], [O])
        assert np.allclose(host(O), oracle.bias_add(x, b), **_tol(dt))
        by_id(f"bias_add_{sfx}_v0", OpKind.BiasAdd, [X, dev(b, dt)], [X])  # in place
        assert np.allclose(host(X), oracle.bias_add(x, b), **_tol(dt))


def test_reference_alias_ids_and_legacy_dispatch(gpu):
    x = oracle.f16_round(rnd((64, 256), 1))
    X, O = dev(x, "f16"), Tensor.empty((64, 256), "f16")
    for kid, kind in [("relu_f16_vec2_v0", OpKind.EltwiseRelu), ("relu_f16_v0", OpKind.EltwiseRelu)]:
        by_id(kid, kind, [X], [O])
        assert np.array_equal(host(O), np.maximum(x, 0))
    op_call(OpKind.EltwiseRelu, [X], [O])  # legacy path picks by priority
    assert np.array_equal(host(O), np.maximum(x, 0))
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # dtype mismatch by id
        by_id("relu_f32_v0", OpKind.EltwiseRelu, [X], [O])
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # shape mismatch
        by_id("relu_f16_v0", OpKind.EltwiseRelu, [X], [Tensor.empty((64, 255), "f16")])
    with pytest.raises(RuntimeError, match="NotImplemented"):
        by_id("batchnorm_fwd_f16_v0", OpKind.BatchNormFwd, [X], [O])
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # sgd output may not alias the gradient
        by_id("sgd_step_f16_v0", OpKind.SgdStep, [X, O], [O])


def test_relu_bwd_covers_sizes_the_reference_truncates(gpu):
    n = 65535 * 256 + 12345  # the reference's grid cap leaves everything past 65535*256 unwritten
    dout = np.ones(n, np.float32)
    y = np.ones(n, np.float32)
    y[::3] = -1
    O = Tensor.from_numpy(np.full(n, 7, np.float32))
    by_id("relu_bwd_f32_v0", OpKind.ReluBwd, [dev(dout), dev(y)], [O])
    got = host(O)
    assert np.array_equal(got, np.where(y > 0, 1, 0).astype(np.float32))


@pytest.mark.parametrize("src,dst", [("f32", "bf16"), ("f32", "f16"), ("bf16", "f32"), ("f16", "bf16")])
def test_cast_rounds_to_nearest_even(gpu, src, dst):
    x = _round(rnd((33, 1001), 9, 3.0), src)
    O = Tensor.empty(x.shape, dst)
    by_id("cast_v0", OpKind.Cast, [dev(x, src)], [O])
    assert np.array_equal(host(O), _round(x, dst))


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("M,N,dt,out", [(128, 64, "f32", "f32"), (257, 64, "f16", "f32"), (257, 64, "f16", "f16"),
                                        (1000, 130, "f32", "f32"), (4099, 1000, "bf16", "f32"), (65536, 96, "f32", "f32"),
                                        (8192, 8192, "bf16", "f32"), (64, 10, "f32", "f32"), (3, 5, "bf16", "bf16")])
def test_column_sum_fixed_order_and_exact_to_tolerance(gpu, M, N, dt, out):
    x = _round(rnd((M, N), 11), dt)
    kid = {("f32", "f32"): "reduce_sum_keep_lastdim_f32_v0", ("f16", "f32"): "reduce_sum_keep_lastdim_f16_to_f32_v0",
           ("f16", "f16"): "reduce_sum_keep_lastdim_f16_v0", ("bf16", "f32"): "reduce_sum_keep_lastdim_bf16_to_f32_v0",
           ("bf16", "bf16"): "reduce_sum_keep_lastdim_bf16_v0"}[(dt, out)]
    X, O = dev(x, dt), Tensor.empty((N,), out)
    by_id(kid, OpKind.ReduceSum, [X], [O], RSUM, struct.pack("<q", 0))
    want = oracle.reduce_sum_columns(x)
    got = host(O)
    l1 = np.abs(x).astype(np.float64).sum(axis=0)
    if out == "f32":
        assert (np.abs(got - want) <= 1e-5 * l1 + 1e-30).all()
    else:
        assert np.allclose(got, want, rtol=8e-3 if out == "bf16" else 1e-3, atol=1e-2)
    by_id(kid, OpKind.ReduceSum, [X], [O])  # no attrs: axis defaults to 0
    assert np.array_equal(host(O), got), "two runs must agree bit for bit (fixed summation order)"
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # the column-sum ids accept axis 0 only
        by_id(kid, OpKind.ReduceSum, [X], [O], RSUM, struct.pack("<q", 1))


def test_column_sum_rank3_flattens_leading_dims(gpu):
    x = rnd((8, 32, 128), 12)
    O = Tensor.empty((128,))
    by_id("reduce_sum_keep_lastdim_f32_v0", OpKind.ReduceSum, [dev(x)], [O])
    assert_close_f32(host(O), oracle.reduce_sum_columns(x), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("M,N", [(256, 4096), (33, 1000), (1, 65536), (17, 1001), (5, 3)])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("kind", ["sum", "max", "mean"])
def test_last_axis_reductions(gpu, M, N, dt, kind):
    x = _round(oracle.softmax_inputs(M, N, seed=2), dt)
    O = Tensor.empty((M,))
    opk = {"sum": OpKind.ReduceSum, "max": OpKind.ReduceMax, "mean": OpKind.ReduceMean}[kind]
    sch, pay = (RSUM, struct.pack("<q", -1)) if kind == "sum" else (0, b"")
    by_id(f"reduce_{kind}_lastaxis_{dt}_v0", opk, [dev(x, dt)], [O], sch, pay)
    want = oracle.reduce_lastaxis(x, kind)
    got = host(O)
    if kind == "max":
        assert np.array_equal(got, want.astype(np.float32))
    else:
        l1 = np.abs(x).astype(np.float64).sum(axis=1) / (N if kind == "mean" else 1)
        assert (np.abs(got - want) <= 1e-5 * l1 + 1e-30).all()
    if kind == "sum":  # legacy dispatch with axis -1 must route to the last-axis kernel, axis 0 to the column sum
        op_call(OpKind.ReduceSum, [dev(x, dt)], [O], RSUM, struct.pack("<q", -1))
        assert np.array_equal(host(O), got)


# ------------------------------------------------------------------ softmax / cross-entropy
@pytest.mark.parametrize("M,N", [(64, 4096), (33, 1000), (8, 32000), (16, 1001), (3, 50000), (128, 8), (5, 32768)])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_softmax_rows(gpu, M, N, dt):
    x = _round(oracle.softmax_inputs(M, N, seed=2), dt)
    Y = Tensor.empty((M, N), dt)
    by_id(f"softmax_lastdim_{dt}_v0", OpKind.Softmax, [dev(x, dt)], [Y])
    assert _C.wait_status() == 0, "a bounded wait of the row prefetch pipeline expired"
    want = oracle.softmax(x)
    got = host(Y)
    if dt == "f32":
        assert_close_f32(got, want, rtol=1e-5, atol=1e-10)
        assert np.allclose(got.astype(np.float64).sum(axis=1), 1, atol=1e-5)
    else:
        assert np.allclose(got, want, rtol=8e-3 if dt == "bf16" else 1e-3, atol=1e-7)
    if dt == "f32":
        assert np.array_equal(np.argmax(got, axis=1), np.argmax(x, axis=1))


@pytest.mark.parametrize("B,Cn", [(64, 32000), (128, 1000), (32, 10), (7, 1001), (4, 40000), (256, 8)])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_softmax_cross_entropy(gpu, B, Cn, dt):
    z, y = oracle.ce_inputs(B, Cn, seed=2)
    z = _round(z, dt)
    D, L, A = Tensor.empty((B, Cn), dt), Tensor.empty((B,)), Tensor.empty((B,), "i32")
    by_id(f"softmax_ce_{dt}_i32_v0", OpKind.SoftmaxCE, [dev(z, dt), dev(y)], [D, L, A])
    assert _C.wait_status() == 0, "a bounded wait of the row prefetch pipeline expired"
    wd, wl, wa = oracle.softmax_ce(z, y)
    assert np.array_equal(A.numpy(), wa), "argmax must be bit-exact"
    assert_close_f32(host(L), wl, rtol=1e-5, atol=1e-6, what="loss rows")
    if dt == "f32":
        assert_close_f32(host(D), wd, rtol=1e-5, atol=1e-12, what="dlogits")
    else:
        # f16 gradients below 6e-5 are subnormal: spacing 6e-8 bounds the absolute error there
        assert np.allclose(host(D), wd, rtol=8e-3 if dt == "bf16" else 1e-3, atol=1e-9 if dt == "bf16" else 6e-8)
    # explicit scale, and the two-output form (no argmax)
    D2, L2 = Tensor.empty((B, Cn), dt), Tensor.empty((B,))
    by_id(f"softmax_ce_{dt}_i32_v0", OpKind.SoftmaxCE, [dev(z, dt), dev(y)], [D2, L2], SMCE, struct.pack("<f", 1.0 / 4096))
    assert np.allclose(host(D2), oracle.softmax_ce(z, y, 1.0 / 4096)[0], rtol=1e-2 if dt != "f32" else 1e-5,
                       atol=6e-8 if dt == "f16" else 1e-12)
    assert np.array_equal(host(L2), host(L))


def test_softmax_ce_ties_and_out_of_range_labels(gpu):
    z = np.zeros((4, 64), np.float32)
    z[0, [5, 9]] = 3.0
    z[1, 63] = 1.0
    y = np.array([5, 64, -1, 0], np.int32)
    D, L, A = Tensor.empty((4, 64)), Tensor.empty((4,)), Tensor.empty((4,), "i32")
    by_id("softmax_ce_f32_i32_v0", OpKind.SoftmaxCE, [dev(z), dev(y)], [D, L, A])
    wd, wl, wa = oracle.softmax_ce(z, y)
    assert list(A.numpy()) == [5, 63, 0, 0] == list(wa)
    assert_close_f32(host(L), wl, atol=1e-6)
    assert_close_f32(host(D), wd, atol=1e-9)


@pytest.mark.parametrize("Cn", [32772, 50000, 65536])
def test_softmax_ce_rows_beyond_one_block_are_split_over_a_cluster(gpu, Cn):
    """fp32 rows of more than 32768 columns do not fit one block's registers: up to 65536 columns a cluster of CTAs
    takes a row, each CTA a slice, and the row is still read once. Ties of the maximum in different slices (the lowest
    column wins), labels in the first and last slice and out of range, against the oracle."""
    B = 6
    z, y = oracle.ce_inputs(B, Cn, seed=5)
    z[0, :] = 0.0
    z[0, [Cn - 1, Cn // 2, 7]] = 4.0          # three-way tie across slices
    z[1, Cn - 1] = 50.0                        # maximum in the last column
    y[:] = [7, Cn - 1, 0, Cn, -3, Cn // 3]     # rows 3 and 4: out of range
    D, L, A = Tensor.empty((B, Cn)), Tensor.empty((B,)), Tensor.empty((B,), "i32")
    by_id("softmax_ce_f32_i32_v0", OpKind.SoftmaxCE, [dev(z), dev(y)], [D, L, A])
    assert _C.wait_status() == 0
    wd, wl, wa = oracle.softmax_ce(z, y)
    assert list(A.numpy()[:2]) == [7, Cn - 1]
    assert np.array_equal(A.numpy(), wa)
    assert_close_f32(host(L), wl, rtol=1e-5, atol=1e-6, what="loss rows")
    assert host(L)[3] == 0.0 and host(L)[4] == 0.0
    assert_close_f32(host(D), wd, rtol=1e-5, atol=1e-12, what="dlogits")
    again = Tensor.empty((B, Cn))
    by_id("softmax_ce_f32_i32_v0", OpKind.SoftmaxCE, [dev(z), dev(y)], [again, L, A])
    assert np.array_equal(host(again), host(D)), "partial sums are added in rank order"


# ------------------------------------------------------------------ multi-tensor Adam (one launch for a whole model)
def _multi_adam(sizes, lp_kinds, step_value, wd, dec, seed=0):
    """Launches adam_step_f32_multi_v1 over tensors of `sizes`; returns per tensor (device results, oracle results)."""
    rng = np.random.default_rng(seed)
    host_in, dev_in, outs, mask = [], [], [], 0
    for t, (n, lpk) in enumerate(zip(sizes, lp_kinds)):
        p = (rng.standard_normal(n) * 0.02).astype(np.float32)
        g = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        m = (rng.standard_normal(n) * 1e-3).astype(np.float32)
        v = np.abs(rng.standard_normal(n) * 1e-6).astype(np.float32)
        host_in.append((p, g, m, v))
        P, G, M, V = dev(p), dev(g), dev(m), dev(v)
        dev_in += [P, G, M, V]
        outs += [P, M, V]
        if lpk:
            outs.append(Tensor.empty((n,), lpk))
            mask |= 1 << t
    step = Tensor.from_numpy(np.array([step_value], np.int32))
    pay = struct.pack("<fffffIII", 3e-4, 0.9, 0.999, 1e-8, wd, dec, len(sizes), mask)
    by_id("adam_step_f32_multi_v1", OpKind.AdamStep, dev_in + [step], outs, ADAM, pay)
    assert _C.wait_status() == 0
    res, k = [], 0
    for t, (n, lpk) in enumerate(zip(sizes, lp_kinds)):
        p, g, m, v = host_in[t]
        want = oracle.adam_step_fused(p, g, m, v, step_value, F(3e-4), F(0.9), F(0.999), F(1e-8), weight_decay=F(wd), decoupled=bool(dec))
        got = [host(outs[k]), host(outs[k + 1]), host(outs[k + 2])]
        k += 3
        lp = None
        if lpk:
            lp = (host(outs[k]), lpk)
            k += 1
        res.append((got, want, lp))
    return res


@pytest.mark.parametrize("wd,dec", [(0.0, 0), (0.01, 0), (0.01, 1)])
def test_adam_multi_tensor_one_launch(gpu, wd, dec):
    # whole 16 KiB chunks, tails of every kind (packets + odd elements), tensors smaller than a chunk, one element
    sizes = [4096 * 37 + 1001, 1000, 8192, 1, 4096 * 5, 4099, 3, 4096 * 301 + 2]
    lps = ["bf16", None, "f16", None, "bf16", "bf16", "f16", None]
    for (got, want, lp), n in zip(_multi_adam(sizes, lps, 7, wd, dec), sizes):
        assert_close_f32(got[0], want[0], what=f"p[{n}]")
        assert_close_f32(got[1], want[1], atol=1e-9, what=f"m[{n}]")
        assert_close_f32(got[2], want[2], atol=1e-13, what=f"v[{n}]")
        if lp:
            assert np.array_equal(lp[0], _round(got[0], lp[1])), f"working copy of the tensor of {n} elements"


def test_adam_multi_tensor_equals_per_tensor_launches_and_checks_its_contract(gpu):
    sizes, lps = [4096 * 9 + 17, 513, 4096 * 2], ["bf16", None, None]
    multi = _multi_adam(sizes, lps, 3, 0.01, 0, seed=5)
    rng = np.random.default_rng(5)
    for (got, _, lp), n, lpk in zip(multi, sizes, lps):  # same draws, one fused launch per tensor: identical bits
        p, g = (rng.standard_normal(n) * 0.02).astype(np.float32), (rng.standard_normal(n) * 1e-3).astype(np.float32)
        m, v = (rng.standard_normal(n) * 1e-3).astype(np.float32), np.abs(rng.standard_normal(n) * 1e-6).astype(np.float32)
        P, G, M, V = dev(p), dev(g), dev(m), dev(v)
        outs = [P, M, V] + ([Tensor.empty((n,), lpk)] if lpk else [])
        by_id("adam_step_f32_fused_v1", OpKind.AdamStep, [P, G, M, V, Tensor.from_numpy(np.array([3], np.int32))], outs, ADAM,
              struct.pack("<fffffI", 3e-4, 0.9, 0.999, 1e-8, 0.01, 0))
        for a, b in zip(got, outs[:3]):
            assert np.array_equal(a, host(b))
        if lpk:
            assert np.array_equal(lp[0], host(outs[3]))
    # contract: in place only, count must match the operand lists, at most 16 tensors
    P, G, M, V = (dev(rnd((64,), i)) for i in range(4))
    step = Tensor.from_numpy(np.array([1], np.int32))
    pay = lambda count, mask: struct.pack("<fffffIII", 1e-3, 0.9, 0.999, 1e-8, 0.0, 0, count, mask)
    with pytest.raises(RuntimeError, match="InvalidArgument"):   # out of place
        by_id("adam_step_f32_multi_v1", OpKind.AdamStep, [P, G, M, V, step], [Tensor.empty((64,)), M, V], ADAM, pay(1, 0))
    with pytest.raises(RuntimeError, match="InvalidArgument"):   # count says two tensors, one is given
        by_id("adam_step_f32_multi_v1", OpKind.AdamStep, [P, G, M, V, step], [P, M, V], ADAM, pay(2, 0))
    with pytest.raises(RuntimeError, match="InvalidArgument"):   # a working copy is announced but not passed
        by_id("adam_step_f32_multi_v1", OpKind.AdamStep, [P, G, M, V, step], [P, M, V], ADAM, pay(1, 1))
    with pytest.raises(RuntimeError, match="InvalidArgument"):   # the plain fused payload is not enough
        by_id("adam_step_f32_multi_v1", OpKind.AdamStep, [P, G, M, V, step], [P, M, V], ADAM,
              struct.pack("<fffffI", 1e-3, 0.9, 0.999, 1e-8, 0.0, 0))
