"""The NumPy oracle against known answers and against plain-Python restatements of the same formulas
(small cases, loops), plus the interpreter on the small MLP configuration. CPU only."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

import oracle
from aicf_cuda import build_mlp_train_step

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_bf16_round_ties_to_even():
    x = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, 1.0 + 2.0 ** -7, -1.0 - 2.0 ** -8, 3.14159], np.float32)
    want = np.array([1.0, 1.0 + 2.0 ** -6, 1.0 + 2.0 ** -7, -1.0, 3.140625], np.float32)
    assert np.array_equal(oracle.bf16_round(x), want)


def test_bf16_bits_roundtrip_matches_package_helper():
    from aicf_cuda import bf16_bits_to_f32, f32_to_bf16_bits
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    assert np.array_equal(bf16_bits_to_f32(f32_to_bf16_bits(x)), oracle.bf16_round(x))


def test_gemm_matches_triple_loop():
    rng = np.random.default_rng(1)
    A, B = rng.standard_normal((3, 4)), rng.standard_normal((4, 5))
    want = [[sum(A[i, k] * B[k, j] for k in range(4)) for j in range(5)] for i in range(3)]
    assert np.allclose(oracle.gemm(A, B), want, rtol=1e-14)
    assert np.allclose(oracle.gemm(A.T.copy(), B, transA=True), want, rtol=1e-14)
    assert np.allclose(oracle.gemm(A, B.T.copy(), transB=True), want, rtol=1e-14)
    bias = rng.standard_normal(5)
    e = oracle.gemm_epilogue(A, B, bias)  # default: relu on
    assert np.allclose(e, np.maximum(np.array(want) + bias, 0))
    assert np.allclose(oracle.gemm_epilogue(A, B, bias, relu=False), np.array(want) + bias)


def test_adam_v0_known_answer_divisor_semantics():
    # one element, by hand: p=1, g=0.5, m=0.1, v=0.2, lr=1e-3, b1=.9, b2=.999, eps=1e-8, bc1=1-.9^3, bc2=1-.999^3
    bc1, bc2 = 1 - 0.9 ** 3, 1 - 0.999 ** 3
    m2 = 0.9 * 0.1 + 0.1 * 0.5
    v2 = 0.999 * 0.2 + 0.001 * 0.25
    p2 = 1.0 - 1e-3 * ((m2 / bc1) / (math.sqrt(v2 / bc2) + 1e-8))
    p, m, v = oracle.adam_step_v0([1.0], [0.5], [0.1], [0.2], bc1, bc2)
    assert p[0] == pytest.approx(p2, rel=1e-15) and m[0] == pytest.approx(m2, rel=1e-15) and v[0] == pytest.approx(v2, rel=1e-15)


def test_adam_fused_equals_v0_fed_with_divisors_and_first_step_is_sign_step():
    rng = np.random.default_rng(3)
    p, g = rng.standard_normal(64), rng.standard_normal(64) * 1e-3
    m, v = np.zeros(64), np.zeros(64)
    a = oracle.adam_step_fused(p, g, m, v, step=1, lr=3e-4)
    b = oracle.adam_step_v0(p, g, m, v, 1 - 0.9, 1 - 0.999, lr=3e-4)
    for x, y in zip(a, b):
        assert np.allclose(x, y, rtol=1e-13)
    # at t=1 with zero state, m_hat = g and v_hat = g^2: the update is lr * g/(|g|+eps)
    assert np.allclose(a[0], p - 3e-4 * g / (np.abs(g) + 1e-8), rtol=1e-9)


def test_adam_weight_decay_modes():
    p, g, z = np.array([2.0]), np.array([0.1]), np.array([0.0])
    coupled = oracle.adam_step_fused(p, g, z, z, 1, weight_decay=0.01)
    same = oracle.adam_step_fused(p, g + 0.01 * p, z, z, 1)
    assert np.allclose(coupled[0], same[0]) and np.allclose(coupled[1], same[1])
    dec = oracle.adam_step_fused(p, g, z, z, 1, lr=1e-3, weight_decay=0.01, decoupled=True)
    plain = oracle.adam_step_fused(p, g, z, z, 1, lr=1e-3)
    assert np.allclose(dec[0], plain[0] - 1e-3 * 0.01 * p)


def test_bias_corr_known_answers_and_clamp():
    b1, b2 = oracle.bias_corr(1)
    assert b1 == pytest.approx(1 / (1 - 0.9)) and b2 == pytest.approx(1 / (1 - 0.999))
    assert oracle.bias_corr(0) == oracle.bias_corr(1)  # t is clamped to >= 1
    b1, b2 = oracle.bias_corr(10, 0.9, 0.999)
    assert b1 == pytest.approx(1 / (1 - 0.9 ** 10)) and b2 == pytest.approx(1 / (1 - 0.999 ** 10))


def test_softmax_ce_matches_loops_and_invariants():
    rng = np.random.default_rng(5)
    z = rng.standard_normal((6, 11)) * 2
    y = rng.integers(0, 11, 6)
    d, loss, am = oracle.softmax_ce(z, y)
    for r in range(6):
        mx = max(z[r])
        se = sum(math.exp(t - mx) for t in z[r])
        assert loss[r] == pytest.approx(math.log(se) + mx - z[r, y[r]], rel=1e-12)
        for c in range(11):
            want = (math.exp(z[r, c] - mx) / se - (1.0 if c == y[r] else 0.0)) / 6
            assert d[r, c] == pytest.approx(want, rel=1e-10, abs=1e-15)
        assert am[r] == int(np.argmax(z[r]))
    assert np.allclose(d.sum(axis=1), 0, atol=1e-15)
    assert (loss >= 0).all()


def test_softmax_ce_argmax_ties_pick_lowest_index_and_bad_labels_are_ignored():
    z = np.array([[1.0, 3.0, 3.0, 0.0], [0.0, 0.0, 0.0, 0.0]])
    d, loss, am = oracle.softmax_ce(z, np.array([7, -1]))
    assert list(am) == [1, 0]
    assert list(loss) == [0.0, 0.0]
    assert np.allclose(d.sum(axis=1), 0.5)  # softmax * scale, no one-hot


def test_reductions_and_elementwise_against_loops():
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, 3, 4))
    assert np.allclose(oracle.reduce_sum_columns(x), [sum(x[i, j, c] for i in range(5) for j in range(3)) for c in range(4)])
    assert np.allclose(oracle.reduce_lastaxis(x, "mean"), x.sum(-1) / 4)
    assert np.array_equal(oracle.reduce_lastaxis(x, "max"), x.max(-1))
    y = rng.standard_normal((5, 3, 4))
    assert np.array_equal(oracle.relu_bwd(x, y), np.where(y > 0, x, 0))
    assert np.allclose(oracle.mse_grad(x, y), (x - y) * 2 / 60)
    assert np.allclose(oracle.sgd_step(x, y), x - 1e-3 * y)
    assert np.array_equal(oracle.step_inc(np.array([4], np.int32)), [5])


def _small_mlp_env(dtype="f32"):
    dims = [784, 256, 10]
    vals, low = build_mlp_train_step(64, dims, compute_dtype=dtype, lr=1e-3)
    params = oracle.mlp_params(dims, seed=0)
    x, y = oracle.mlp_batch(64, 784, 10, seed=0)
    env, dtypes = {}, {}
    for v in vals:
        dtypes[v.vid] = v.dtype
        if v.name == "x":
            env[v.vid] = x
        elif v.name == "labels":
            env[v.vid] = y
        elif v.name in params:
            env[v.vid] = params[v.name].copy()
        elif v.name.endswith(".lp"):
            env[v.vid] = oracle.cast(params[v.name[:-3]], v.dtype) if v.name[:-3] in params else np.zeros(v.shape, np.float32)
        else:
            env[v.vid] = np.zeros(v.shape, np.int32 if v.dtype == "i32" else np.float32)
    return vals, low, env, dtypes


def test_interpreter_trains_the_small_mlp():
    vals, low, env, dtypes = _small_mlp_env()
    by = {v.name: v.vid for v in vals}
    losses = []
    for _ in range(10):
        oracle.run_lowered(low, env, dtypes, np.float64)
        losses.append(float(env[by["loss"]][0]))
    assert losses[0] == pytest.approx(math.log(10), abs=1.0)  # random He init: a little above ln(10)
    assert all(b < a for a, b in zip(losses, losses[1:]))      # same batch every step: loss must fall
    assert int(env[by["opt.step"]][0]) == 10


def test_interpreter_fp32_tracks_fp64():
    _, low, e64, dtypes = _small_mlp_env()
    vals, _, e32, _ = _small_mlp_env()
    by = {v.name: v.vid for v in vals}
    for _ in range(3):
        oracle.run_lowered(low, e64, dtypes, np.float64)
        oracle.run_lowered(low, e32, dtypes, np.float32)
    assert abs(e64[by["loss"]][0] - e32[by["loss"]][0]) < 1e-4
    assert np.allclose(e64[by["0.W"]], e32[by["0.W"]], atol=2e-4)


def test_oracle_against_reference_cuda_golden_vectors():
    """Outputs of the reference's own CUDA kernels (built by oracle/ref_build.py and run on a B200 by
    tests/golden/make_ref_golden.py) pin the restatement of every op the reference implements."""
    path = GOLDEN / "ref_cuda_golden.npz"
    if not path.exists():
        pytest.skip("reference golden vectors have not been generated yet")
    g = np.load(path)
    A, B, bias = g["gemm_A"], g["gemm_B"], g["gemm_bias"]
    for ta in (0, 1):
        for tb in (0, 1):
            a = A.T.copy() if ta else A
            b = B.T.copy() if tb else B
            assert np.allclose(oracle.gemm(a, b, ta, tb), g[f"gemm_f32_{ta}{tb}"], rtol=1e-5, atol=1e-5)
            for relu in (0, 1):
                assert np.allclose(oracle.gemm_epilogue(a, b, bias, ta, tb, relu), g[f"gemm_epi_f32_{ta}{tb}{relu}"], rtol=1e-5, atol=1e-5)
    x, y = g["elt_x"], g["elt_y"]
    assert np.array_equal(oracle.relu(x, np.float32), g["relu_f32"])
    assert np.array_equal(oracle.relu_bwd(x, y, np.float32), g["relu_bwd_f32"])
    assert np.allclose(oracle.mse_grad(x, y), g["mse_grad_f32"], rtol=1e-6, atol=1e-9)
    assert np.allclose(oracle.add(x, y), g["add_f32"], rtol=1e-7)
    assert np.allclose(oracle.sgd_step(x, y), g["sgd_f32"], rtol=1e-6, atol=1e-9)
    assert np.allclose(oracle.bias_add(x, g["elt_bias"]), g["bias_add_f32"], rtol=1e-7)
    assert np.allclose(oracle.reduce_sum_columns(g["red_x"]), g["colsum_f32"], rtol=1e-5, atol=1e-5)
    f = np.float32  # the kernels receive their hyper-parameters as float32
    p, m, v = oracle.adam_step_v0(g["adam_p"], g["adam_g"], g["adam_m"], g["adam_v"], g["adam_bc"][0], g["adam_bc"][1],
                                  f(1e-3), f(0.9), f(0.999), f(1e-8))
    assert np.allclose(p, g["adam_p_out"], rtol=1e-6, atol=1e-8) and np.allclose(m, g["adam_m_out"], rtol=1e-6, atol=1e-9)
    assert np.allclose(v, g["adam_v_out"], rtol=1e-6, atol=1e-12)
    for t in (1, 10):
        b1, b2 = oracle.bias_corr(t, f(0.9), f(0.999))
        assert np.allclose([b1, b2], g[f"bias_corr_{t}"], rtol=1e-4)  # the reference's fp32 powf: 1-0.999^t cancels
    # layer norm (mean offset 0.5, std 2: the reference's one-pass variance loses ~1e-7 relative here)
    assert "ln_x" in g.files, "regenerate tests/golden/ref_cuda_golden.npz with tests/golden/make_ref_golden.py"
    lx, ldy, lg, lb = g["ln_x"], g["ln_dy"], g["ln_gamma"], g["ln_beta"]
    yy, mu, rs = oracle.layernorm_fwd(lx, lg, lb, f(1e-5))
    assert np.allclose(mu, g["ln_mean"], rtol=1e-5, atol=1e-6) and np.allclose(rs, g["ln_rstd"], rtol=1e-5)
    assert np.allclose(yy, g["ln_y_affine"], rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.layernorm_fwd(lx, None, None, f(1e-5))[0], g["ln_y_plain"], rtol=1e-5, atol=1e-5)
    dx, dg, db = oracle.layernorm_bwd(lx, ldy, lg, g["ln_mean"], g["ln_rstd"])
    assert np.allclose(dx, g["ln_dx_affine"], rtol=1e-5, atol=1e-5)
    assert np.allclose(dg, g["ln_dgamma"], rtol=1e-5, atol=1e-5) and np.allclose(db, g["ln_dbeta"], rtol=1e-5, atol=1e-5)
    assert np.allclose(oracle.layernorm_bwd(lx, ldy, None, g["ln_mean"], g["ln_rstd"])[0], g["ln_dx_plain"], rtol=1e-5, atol=1e-5)


def _f16_ulps(got, want):
    """Largest distance in units of the f16 spacing at `want` (normal range floor 2^-14)."""
    want, got = np.asarray(want, np.float64), np.asarray(got, np.float64)
    return float(np.max(np.abs(got - want) / (np.maximum(np.abs(want), 2.0 ** -14) * 2.0 ** -10)))


def test_oracle_against_reference_cuda_f16_golden_vectors():
    """The f16 variants of the reference's kernels (same generator, arrays prefixed h_): the oracle computes in fp64
    and rounds once to f16; the reference computes in half2 or fp32 and rounds. Exact where the operation is exactly
    representable before the rounding, one f16 spacing otherwise (two roundings in mse_grad, fp32 accumulation in the
    wmma GEMM and in layer norm)."""
    g = np.load(GOLDEN / "ref_cuda_golden.npz")
    assert "h_x" in g.files, "regenerate tests/golden/ref_cuda_golden.npz with tests/golden/make_ref_golden.py"
    r16 = oracle.f16_round
    x, y = g["h_x"], g["h_y"]
    assert np.array_equal(g["h_relu"], oracle.relu(x)) and np.array_equal(g["h_relu_bwd"], oracle.relu_bwd(x, y))
    assert np.array_equal(g["h_add"], r16(oracle.add(x, y)))
    assert np.array_equal(g["h_sgd"], r16(oracle.sgd_step(x, y)))
    assert np.array_equal(g["h_bias_add"], r16(oracle.bias_add(x, g["h_bias"])))
    assert _f16_ulps(g["h_mse_grad"], r16(oracle.mse_grad(x, y))) <= 1.0
    assert np.array_equal(g["h_colsum_f16"], r16(oracle.reduce_sum_columns(g["h_red_x"])))
    assert np.allclose(g["h_colsum_f32"], oracle.reduce_sum_columns(g["h_red_x"]), rtol=1e-6, atol=1e-5)
    A, B, bias = g["h_gemm_A"], g["h_gemm_B"], g["h_gemm_bias"]
    for ta in (0, 1):
        for tb in (0, 1):
            a = A.T.copy() if ta else A
            b = B.T.copy() if tb else B
            assert _f16_ulps(g[f"h_gemm_{ta}{tb}"], r16(oracle.gemm(a, b, ta, tb))) <= 1.0
            assert _f16_ulps(g[f"h_gemm_epi_{ta}{tb}"], r16(oracle.gemm_epilogue(a, b, bias, ta, tb, 1))) <= 1.0
    yy, mu, rs = oracle.layernorm_fwd(g["h_ln_x"], g["h_ln_gamma"], g["h_ln_beta"], np.float32(1e-5))
    assert _f16_ulps(g["h_ln_y"], r16(yy)) <= 1.0
    assert np.allclose(mu, g["h_ln_mean"], rtol=1e-5, atol=1e-6) and np.allclose(rs, g["h_ln_rstd"], rtol=1e-5)
    dx, dgam, dbet = oracle.layernorm_bwd(g["h_ln_x"], g["h_ln_dy"], g["h_ln_gamma"], g["h_ln_mean"], g["h_ln_rstd"])
    assert _f16_ulps(g["h_ln_dx"], r16(dx)) <= 1.0
    assert np.allclose(dgam, g["h_ln_dgamma"], rtol=1e-5, atol=1e-5) and np.allclose(dbet, g["h_ln_dbeta"], rtol=1e-5, atol=1e-5)
