"""Our kernels against the REFERENCE's own CUDA kernels (its unmodified sources compiled into
oracle/_ref/libaicf_ref.so by oracle/ref_build.py), on the same device buffers, for every op the
reference implements on this path. fp32: 1e-5 relative; integer outputs exact; f16 tensor-core GEMM:
both are compared with fp64 and with each other at one f16 rounding."""
import struct

import numpy as np
import pytest

import oracle
from aicf_cuda import Tensor
from aicf_cuda._C import OpKind
from util import assert_close_f32, by_id, dev, host, ref_by_id, rel_err

pytestmark = pytest.mark.gpu

SHAPES = [(1024,), (64, 256), (8, 32, 128)]


def rnd(shape, seed=0, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def both(ref_lib, kid, kind, ins, out_shapes, out_dtypes, schema=0, payload=b"", expect_ok=True):
    ours = [Tensor.zeros(s, d) for s, d in zip(out_shapes, out_dtypes)]
    theirs = [Tensor.zeros(s, d) for s, d in zip(out_shapes, out_dtypes)]
    st = ref_by_id(ref_lib, kid, kind, ins, theirs, schema, payload)
    assert (st == 0) == expect_ok, f"reference status {st}"
    by_id(kid, kind, ins, ours, schema, payload)
    return ours, theirs


@pytest.mark.parametrize("shape", SHAPES)
def test_elementwise_f32_bit_exact_vs_reference(ref_lib, shape):
    x, y = rnd(shape, 1), rnd(shape, 2)
    X, Y = dev(x), dev(y)
    for kid, kind, ins in [("relu_f32_v0", OpKind.EltwiseRelu, [X]), ("relu_bwd_f32_v0", OpKind.ReluBwd, [X, Y]),
                           ("add_f32_v0", OpKind.EltwiseAdd, [X, Y]), ("copy_f32_v0", OpKind.Copy, [X]),
                           ("mse_grad_f32_v0", OpKind.MseGrad, [X, Y]), ("sgd_step_f32_v0", OpKind.SgdStep, [X, Y])]:
        o, t = both(ref_lib, kid, kind, ins, [shape], ["f32"])
        assert_close_f32(host(o[0]), host(t[0]), rtol=1e-6, atol=1e-9, what=kid)
    if len(shape) >= 2:
        b = dev(rnd((shape[-1],), 3))
        o, t = both(ref_lib, "bias_add_f32_v0", OpKind.BiasAdd, [X, b], [shape], ["f32"])
        assert np.array_equal(host(o[0]), host(t[0]))


@pytest.mark.parametrize("shape", [(7, 33, 127), (64, 256)])
def test_elementwise_f16_vs_reference(ref_lib, shape):
    x, y = oracle.f16_round(rnd(shape, 1)), oracle.f16_round(rnd(shape, 2))
    X, Y = dev(x, "f16"), dev(y, "f16")
    for kid, kind, ins in [("relu_f16_v0", OpKind.EltwiseRelu, [X]), ("relu_bwd_f16_v0", OpKind.ReluBwd, [X, Y]),
                           ("add_f16_v0", OpKind.EltwiseAdd, [X, Y]), ("copy_f16_v0", OpKind.Copy, [X]),
                           ("sgd_step_f16_v0", OpKind.SgdStep, [X, Y]), ("mse_grad_f16_v0", OpKind.MseGrad, [X, Y])]:
        o, t = both(ref_lib, kid, kind, ins, [shape], ["f16"])
        assert np.allclose(host(o[0]), host(t[0]), rtol=1e-3, atol=1e-7), kid


@pytest.mark.parametrize("M,K,N", [(64, 48, 80), (128, 64, 256)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_f32_bit_exact_vs_reference(ref_lib, M, K, N, ta, tb):
    A, B, bias = oracle.gemm_inputs(M, N, K, seed=1)
    sa = dev(np.ascontiguousarray(A.T) if ta else A)
    sb = dev(np.ascontiguousarray(B.T) if tb else B)
    o, t = both(ref_lib, "gemm_f32_naive_v0", OpKind.Gemm, [sa, sb], [(M, N)], ["f32"], 0x47454D4D, struct.pack("<ii", ta, tb))
    assert np.array_equal(host(o[0]), host(t[0])), "same FMA order => same bits"
    for relu in (1, 0):
        o, t = both(ref_lib, "gemm_bias_relu_f32_naive_v0", OpKind.GemmEpilogue, [sa, sb, dev(bias)], [(M, N)], ["f32"],
                    0x4750454C, struct.pack("<iii", ta, tb, relu))
        assert_close_f32(host(o[0]), host(t[0]), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_f16_vs_reference_wmma(ref_lib, ta, tb):
    M = N = K = 64
    A, B, bias = oracle.gemm_inputs(M, N, K, seed=1)
    A, B, bias = oracle.f16_round(A), oracle.f16_round(B), oracle.f16_round(bias)
    sa = dev(np.ascontiguousarray(A.T) if ta else A, "f16")
    sb = dev(np.ascontiguousarray(B.T) if tb else B, "f16")
    o, t = both(ref_lib, "gemm_f16_tc_wmma_out_f16_v0", OpKind.Gemm, [sa, sb], [(M, N)], ["f16"], 0x47454D4D, struct.pack("<ii", ta, tb))
    want = oracle.gemm(A, B)
    assert rel_err(host(t[0]), want) <= 2e-2 and rel_err(host(o[0]), want) <= 2e-2
    assert rel_err(host(o[0]), host(t[0])) <= 2e-3
    o, t = both(ref_lib, "gemm_bias_relu_f16_tc_wmma_out_f16_v0", OpKind.GemmEpilogue, [sa, sb, dev(bias, "f16")], [(M, N)], ["f16"],
                0x4750454C, struct.pack("<iii", ta, tb, 1))
    assert rel_err(host(o[0]), host(t[0])) <= 2e-3


@pytest.mark.parametrize("M,N,dt,out,kid", [(128, 64, "f32", "f32", "reduce_sum_keep_lastdim_f32_v0"),
                                            (257, 64, "f16", "f32", "reduce_sum_keep_lastdim_f16_to_f32_v0"),
                                            (4096, 256, "f32", "f32", "reduce_sum_keep_lastdim_f32_v0")])
def test_column_sum_vs_reference(ref_lib, M, N, dt, out, kid):
    x = rnd((M, N), 11)
    x = oracle.f16_round(x) if dt == "f16" else x
    o, t = both(ref_lib, kid, OpKind.ReduceSum, [dev(x, dt)], [(N,)], [out])
    l1 = np.abs(x).astype(np.float64).sum(axis=0)
    assert (np.abs(host(o[0]).astype(np.float64) - host(t[0])) <= 1e-5 * l1).all()
    st = ref_by_id(ref_lib, kid, OpKind.ReduceSum, [dev(x, dt)], [Tensor.empty((N,), out)], 0x5253554D, struct.pack("<q", 1))
    assert st == 1  # the reference also answers InvalidArgument for axis 1


@pytest.mark.parametrize("shape", SHAPES)
def test_adam_step_vs_reference(ref_lib, shape):
    p, g, m, v = rnd(shape, 1), rnd(shape, 2, 1e-2), rnd(shape, 3, 1e-2), np.abs(rnd(shape, 4, 1e-3))
    sc = [Tensor.from_numpy(np.array(1 - 0.9 ** 3, np.float32)), Tensor.from_numpy(np.array(1 - 0.999 ** 3, np.float32))]
    ins = [dev(p), dev(g), dev(m), dev(v)] + sc
    o, t = both(ref_lib, "adam_step_f32_v0", OpKind.AdamStep, ins, [shape] * 3, ["f32"] * 3, 0x4D414441,
                struct.pack("<ffff", 1e-3, 0.9, 0.999, 1e-8))
    for a, b, name in zip(o, t, "pmv"):
        assert_close_f32(host(a), host(b), rtol=1e-5, atol=1e-12, what=name)


def test_bias_corr_and_step_inc_vs_reference(ref_lib):
    for step in (1, 10, 0):
        S = Tensor.from_numpy(np.array(step, np.int32))
        o, t = both(ref_lib, "bias_corr_v0", OpKind.BiasCorr, [S], [(), ()], ["f32", "f32"], 0x524F4342, struct.pack("<ff", 0.9, 0.999))
        assert np.array_equal(host(o[0]), host(t[0])) and np.array_equal(host(o[1]), host(t[1]))
    S = Tensor.from_numpy(np.arange(1024, dtype=np.int32))
    ours, theirs = Tensor.from_numpy(np.arange(1024, dtype=np.int32)), Tensor.from_numpy(np.arange(1024, dtype=np.int32))
    assert ref_by_id(ref_lib, "step_inc_v0", OpKind.StepInc, [S], [theirs]) == 0
    by_id("step_inc_v0", OpKind.StepInc, [S], [ours])
    assert np.array_equal(ours.numpy(), theirs.numpy())
