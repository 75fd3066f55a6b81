"""GEMM / GEMM+bias+ReLU parity: tcgen05 kernel (bf16 / f16) and SIMT kernel (f32, unaligned shapes),
all four transpose combinations, ragged edges, strided outputs. Tolerance: 16-bit inputs within 2e-2
relative (normwise) of an fp64 host result - in practice ~4e-3, one rounding of the 16-bit output;
fp32 within 1e-5."""
import struct

import numpy as np
import pytest

import oracle
from aicf_cuda import _C, Tensor
from aicf_cuda._C import OpKind
from util import by_id, dev, gemm_tuning, host, op_call, rel_err

pytestmark = pytest.mark.gpu

GEMM = 0x47454D4D
GPEL = 0x4750454C

_ROUND = {"bf16": oracle.bf16_round, "f16": oracle.f16_round, "f32": lambda a: np.asarray(a, np.float32)}


def _operands(M, N, K, ta, tb, dt, seed=1):
    A, B, bias = oracle.gemm_inputs(M, N, K, seed)
    A, B = _ROUND[dt](A), _ROUND[dt](B)
    sa = np.ascontiguousarray(A.T) if ta else A   # stored [K,M] when transA
    sb = np.ascontiguousarray(B.T) if tb else B   # stored [N,K] when transB
    return A, B, bias, sa, sb


GEMM_KID = {("bf16", "bf16"): "gemm_bf16_tcgen05_out_bf16_v0", ("bf16", "f32"): "gemm_bf16_tcgen05_out_f32_v0",
            ("f16", "f16"): "gemm_f16_tcgen05_out_f16_v0", ("f16", "f32"): "gemm_f16_tcgen05_out_f32_v0",
            ("f32", "f32"): "gemm_f32_naive_v0"}
EPI_KID = {("bf16", "bf16"): "gemm_bias_relu_bf16_tcgen05_out_bf16_v0", ("bf16", "f32"): "gemm_bias_relu_bf16_tcgen05_out_f32_v0",
           ("f16", "f16"): "gemm_bias_relu_f16_tcgen05_out_f16_v0", ("f32", "f32"): "gemm_bias_relu_f32_naive_v0"}
TOL = {"bf16": 2e-2, "f16": 2e-2, "f32": 1e-5}

@pytest.fixture(params=["1:256", "1:128", "1:64", "2"], ids=["cta1_n256", "cta1_n128", "cta1_n64", "cta2"])
def cta_group(request):
    """Runs a test with one CTA per tile at each tile width (256, 128, 64 columns) and with CTA pairs (tcgen05
    cta_group::2); without the overrides the launcher picks by tile count."""
    group, _, width = request.param.partition(":")
    with gemm_tuning(cta_group=group, tile_n=width or None):
        yield request.param


SHAPES = [(64, 80, 48), (128, 256, 64), (256, 512, 128), (200, 304, 136), (1, 8, 8), (129, 257, 72), (384, 1000, 512),
          (1024, 1024, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("dt,out", [("bf16", "bf16"), ("bf16", "f32"), ("f16", "f16"), ("f32", "f32")])
def test_gemm_all_transposes(gpu, cta_group, M, N, K, ta, tb, dt, out):
    # operands whose rows are not 16-byte aligned route to the SIMT kernel inside the same variant
    A, B, _, sa, sb = _operands(M, N, K, ta, tb, dt)
    C = Tensor.empty((M, N), out)
    by_id(GEMM_KID[(dt, out)], OpKind.Gemm, [dev(sa, dt), dev(sb, dt)], [C], GEMM, struct.pack("<ii", ta, tb))
    assert _C.gemm_status() == 0
    want = oracle.gemm(A, B)
    assert rel_err(host(C), want) <= (TOL[dt] if out != "f32" or dt == "f32" else 1e-4), (M, N, K, ta, tb, dt, out)


@pytest.mark.parametrize("M,N,K", [(64, 80, 48), (256, 512, 128), (200, 304, 136), (777, 1000, 264)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("relu", [1, 0])
@pytest.mark.parametrize("dt,out,bias_dt", [("bf16", "bf16", "f32"), ("bf16", "bf16", "bf16"), ("f16", "f16", "f32"),
                                            ("bf16", "f32", "f32"), ("f32", "f32", "f32")])
def test_gemm_epilogue_bias_relu(gpu, cta_group, M, N, K, ta, tb, relu, dt, out, bias_dt):
    A, B, bias, sa, sb = _operands(M, N, K, ta, tb, dt)
    bias = _ROUND[bias_dt](bias)
    C = Tensor.empty((M, N), out)
    by_id(EPI_KID[(dt, out)], OpKind.GemmEpilogue, [dev(sa, dt), dev(sb, dt), dev(bias, bias_dt)], [C], GPEL,
          struct.pack("<iii", ta, tb, relu))
    assert _C.gemm_status() == 0
    want = oracle.gemm_epilogue(A, B, bias, relu=bool(relu))
    assert rel_err(host(C), want) <= (TOL[dt] if out != "f32" or dt == "f32" else 1e-4)
    if relu:
        assert (host(C) >= 0).all()


@pytest.mark.parametrize("M,N,K", [(64, 80, 48), (256, 512, 128), (200, 304, 136), (129, 257, 72), (512, 1024, 1000)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1)])
@pytest.mark.parametrize("dt", ["bf16", "f16", "f32"])
def test_gemm_with_relu_backward_mask(gpu, cta_group, M, N, K, ta, tb, dt):
    """dX = (Y > 0) ? dY*op(W) : 0 in one kernel == the reference's gemm followed by relu_bwd."""
    A, B, _, sa, sb = _operands(M, N, K, ta, tb, dt)
    y = _ROUND[dt](np.random.default_rng(7).standard_normal((M, N)).astype(np.float32))
    y[::3, ::5] = 0.0
    y[1, 1] = np.nan
    kid = {"bf16": "gemm_relu_bwd_bf16_tcgen05_out_bf16_v0", "f16": "gemm_relu_bwd_f16_tcgen05_out_f16_v0", "f32": "gemm_relu_bwd_f32_v0"}[dt]
    C = Tensor.empty((M, N), dt)
    by_id(kid, OpKind.GemmReluBwd, [dev(sa, dt), dev(sb, dt), dev(y, dt)], [C], GEMM, struct.pack("<ii", ta, tb))
    assert _C.gemm_status() == 0
    got = host(C)
    want = oracle.gemm_relu_bwd(A, B, np.nan_to_num(y, nan=-1.0))  # NaN > 0 is false: masked
    assert rel_err(got, want) <= TOL[dt]
    assert not got[~(y > 0)].any(), "every element whose activation is not positive must be exactly zero"
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # the mask must have the output's shape
        by_id(kid, OpKind.GemmReluBwd, [dev(sa, dt), dev(sb, dt), dev(y[:, :-8].copy(), dt)], [C], GEMM, struct.pack("<ii", ta, tb))


def test_reference_ids_keep_reference_contracts(gpu):
    """gemm_f16_tc_wmma_out_f16_v0 / gemm_bias_relu_f16_tc_wmma_out_f16_v0: f16 everything (bias too),
    packed row-major C; schema 0 means no transposes and, for the epilogue, ReLU on."""
    M, N, K = 64, 64, 64
    A, B, bias, sa, sb = _operands(M, N, K, 0, 0, "f16")
    bias = oracle.f16_round(bias)
    C = Tensor.empty((M, N), "f16")
    by_id("gemm_f16_tc_wmma_out_f16_v0", OpKind.Gemm, [dev(sa, "f16"), dev(sb, "f16")], [C])
    assert rel_err(host(C), oracle.gemm(A, B)) <= 2e-2
    by_id("gemm_bias_relu_f16_tc_wmma_out_f16_v0", OpKind.GemmEpilogue, [dev(sa, "f16"), dev(sb, "f16"), dev(bias, "f16")], [C])
    assert rel_err(host(C), oracle.gemm_epilogue(A, B, bias, relu=True)) <= 2e-2
    # a payload under the executor's 'GEPI' tag is ignored exactly like the reference does: ta=tb=0, relu on
    by_id("gemm_bias_relu_f16_tc_wmma_out_f16_v0", OpKind.GemmEpilogue, [dev(sa, "f16"), dev(sb, "f16"), dev(bias, "f16")],
          [C], int.from_bytes(b"GEPI", "little"), struct.pack("<iii", 0, 1, 1))
    assert rel_err(host(C), oracle.gemm_epilogue(A, B, bias, relu=True)) <= 2e-2
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # f32 bias is not this id's contract
        by_id("gemm_bias_relu_f16_tc_wmma_out_f16_v0", OpKind.GemmEpilogue, [dev(sa, "f16"), dev(sb, "f16"), dev(bias)], [C])
    with pytest.raises(RuntimeError, match="InvalidArgument"):  # wrong C shape
        by_id("gemm_f16_tc_wmma_out_f16_v0", OpKind.Gemm, [dev(sa, "f16"), dev(sb, "f16")], [Tensor.empty((M, N + 8), "f16")])
    op_call(OpKind.Gemm, [dev(sa, "f16"), dev(sb, "f16")], [C])  # legacy dispatch finds an f16 variant
    assert rel_err(host(C), oracle.gemm(A, B)) <= 2e-2


def test_f32_matches_sequential_fma_order(gpu):
    """One FMA per k in increasing k, like the reference's fp32 kernel: compare with a float32 loop."""
    M, N, K = 8, 16, 300
    A, B, _ = oracle.gemm_inputs(M, N, K, seed=5)
    C = Tensor.empty((M, N))
    by_id("gemm_f32_naive_v0", OpKind.Gemm, [dev(A), dev(B)], [C])
    acc = np.zeros((M, N), np.float64)
    for k in range(K):  # float32 FMA == round(fp64 product-sum) for these magnitudes
        acc = (acc + A[:, k:k + 1].astype(np.float64) * B[k:k + 1, :].astype(np.float64)).astype(np.float32).astype(np.float64)
    assert np.array_equal(host(C), acc.astype(np.float32))


@pytest.mark.parametrize("size", [4096, 8192])
def test_large_bf16_gemm_sampled_rows(gpu, cta_group, size):
    """Full benchmark sizes: 64 sampled rows against fp64, plus linearity C(2A) == 2 C(A) on the device."""
    M = N = K = size
    rng = np.random.default_rng(1)
    A = oracle.bf16_round(rng.uniform(-1, 1, (M, K)).astype(np.float32))
    B = oracle.bf16_round(rng.uniform(-1, 1, (K, N)).astype(np.float32))
    bias = rng.standard_normal(N).astype(np.float32)
    dA, dB, dbias = dev(A, "bf16"), dev(B, "bf16"), dev(bias)
    C = Tensor.empty((M, N), "bf16")
    by_id("gemm_bias_relu_bf16_tcgen05_out_bf16_v0", OpKind.GemmEpilogue, [dA, dB, dbias], [C], GPEL, struct.pack("<iii", 0, 0, 1))
    assert _C.gemm_status() == 0
    got = host(C)
    rows = rng.choice(M, 64, replace=False)
    want = np.maximum(A[rows].astype(np.float64) @ B.astype(np.float64) + bias, 0)
    assert rel_err(got[rows], want) <= 2e-2
    C2 = Tensor.empty((M, N), "f32")
    C1 = Tensor.empty((M, N), "f32")
    by_id("gemm_bf16_tcgen05_out_f32_v0", OpKind.Gemm, [dA, dB], [C1], GEMM, struct.pack("<ii", 0, 0))
    by_id("gemm_bf16_tcgen05_out_f32_v0", OpKind.Gemm, [dev(2 * A, "bf16"), dB], [C2], GEMM, struct.pack("<ii", 0, 0))
    assert np.array_equal(host(C2), 2 * host(C1)), "scaling an operand by 2 is exact in bf16/fp32"


def test_f32_4096_sampled_rows(gpu):
    n = 4096
    A, B, bias = oracle.gemm_inputs(n, n, n, seed=1)
    C = Tensor.empty((n, n))
    by_id("gemm_bias_relu_f32_naive_v0", OpKind.GemmEpilogue, [dev(A), dev(B), dev(bias)], [C], GPEL, struct.pack("<iii", 0, 0, 1))
    rows = np.random.default_rng(0).choice(n, 32, replace=False)
    want = np.maximum(A[rows].astype(np.float64) @ B.astype(np.float64) + bias, 0)
    assert rel_err(host(C)[rows], want) <= 1e-5


# ------------------------------------------------------------------ fp32 on the tensor cores (3xTF32, opt-in ids)
def _tf32x3_tol(K):
    """Normwise error bound of the 3xTF32 path against fp64: 1e-5, the tolerance of the fp32 ops, for every K. The
    split loses 2^-22 per product; the tensor core's accumulator rounds toward zero at every k step, which the kernel
    confines to chunks of 256 (measured 2.2e-6 at K = 256, 2.0e-6 at 1024, 1.6e-6 at 4096; exact fp32 is at 4e-7)."""
    return 1e-5


@pytest.mark.parametrize("M,N,K", SHAPES + [(130, 70, 50), (64, 200, 37), (1, 1, 1), (300, 129, 1001)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_f32_3xtf32_all_transposes(gpu, M, N, K, ta, tb):
    A, B, bias, sa, sb = _operands(M, N, K, ta, tb, "f32")
    C = Tensor.zeros((M, N), "f32")
    by_id("gemm_f32_3xtf32_v0", OpKind.Gemm, [dev(sa), dev(sb)], [C], GEMM, struct.pack("<ii", ta, tb))
    assert rel_err(host(C), oracle.gemm(A, B)) <= _tf32x3_tol(K)
    for relu in (1, 0):
        by_id("gemm_bias_relu_f32_3xtf32_v0", OpKind.GemmEpilogue, [dev(sa), dev(sb), dev(bias)], [C], GPEL,
              struct.pack("<iii", ta, tb, relu))
        assert rel_err(host(C), oracle.gemm_epilogue(A, B, bias, False, False, bool(relu))) <= _tf32x3_tol(K)
    assert _C.gemm_status() == 0


def test_gemm_f32_3xtf32_is_opt_in_and_much_closer_than_one_tf32_pass(gpu):
    M = N = 256
    K = 512
    A, B, bias, sa, sb = _operands(M, N, K, 0, 1, "f32")
    exact, fast = Tensor.zeros((M, N)), Tensor.zeros((M, N))
    # priority dispatch keeps choosing the exact kernel for fp32 operands
    op_call(OpKind.Gemm, [dev(sa), dev(sb)], [exact], GEMM, struct.pack("<ii", 0, 1))
    ref = Tensor.zeros((M, N))
    by_id("gemm_f32_naive_v0", OpKind.Gemm, [dev(sa), dev(sb)], [ref], GEMM, struct.pack("<ii", 0, 1))
    assert np.array_equal(host(exact), host(ref))
    by_id("gemm_f32_3xtf32_v0", OpKind.Gemm, [dev(sa), dev(sb)], [fast], GEMM, struct.pack("<ii", 0, 1))
    want = oracle.gemm(A, B)
    tf32 = lambda a: (np.asarray(a, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    one_pass = tf32(A).astype(np.float64) @ tf32(B).astype(np.float64)
    assert rel_err(host(fast), want) <= _tf32x3_tol(K) < 0.05 * rel_err(one_pass, want)
    # 16-bit operands are not this id's contract
    with pytest.raises(RuntimeError, match="InvalidArgument"):
        by_id("gemm_f32_3xtf32_v0", OpKind.Gemm, [dev(oracle.f16_round(sa), "f16"), dev(oracle.f16_round(sb), "f16")],
              [Tensor.zeros((M, N), "f16")], GEMM, struct.pack("<ii", 0, 1))
    # the result does not depend on the run
    again = Tensor.zeros((M, N))
    by_id("gemm_f32_3xtf32_v0", OpKind.Gemm, [dev(sa), dev(sb)], [again], GEMM, struct.pack("<ii", 0, 1))
    assert np.array_equal(host(again), host(fast))


def test_gemm_f32_3xtf32_4096_sampled_rows(gpu):
    n = 4096
    A, B, bias = oracle.gemm_inputs(n, n, n, seed=1)
    C = Tensor.empty((n, n))
    by_id("gemm_bias_relu_f32_3xtf32_v0", OpKind.GemmEpilogue, [dev(A), dev(B), dev(bias)], [C], GPEL, struct.pack("<iii", 0, 0, 1))
    rows = np.random.default_rng(0).choice(n, 32, replace=False)
    want = np.maximum(A[rows].astype(np.float64) @ B.astype(np.float64) + bias, 0)
    assert rel_err(host(C)[rows], want) <= _tf32x3_tol(n)
    assert _C.gemm_status() == 0


# ------------------------------------------------------------------ split-K (few tiles, long K)
@pytest.fixture(params=["auto", "3", "8"], ids=["split_auto", "split3", "split8"])
def splitk(request):
    """The launcher's own choice, and forced part counts (3 leaves a ragged last part)."""
    with gemm_tuning(splitk=None if request.param == "auto" else request.param):
        yield request.param


@pytest.mark.parametrize("M,N,K", [(16, 512, 4096), (128, 1024, 8192), (200, 768, 4104), (64, 1000, 5000), (1, 256, 4096)])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("dt,out", [("bf16", "bf16"), ("bf16", "f32"), ("f16", "f16")])
def test_gemm_split_over_k(gpu, splitk, M, N, K, ta, tb, dt, out):
    if ta and M % 8:
        pytest.skip("a transposed A needs 16-byte aligned columns on the tensor-core path")
    A, B, bias, sa, sb = _operands(M, N, K, ta, tb, dt)
    X, W, Bv = dev(sa, dt), dev(sb, dt), dev(bias)
    C = Tensor.zeros((M, N), out)
    by_id(GEMM_KID[(dt, out)], OpKind.Gemm, [X, W], [C], GEMM, struct.pack("<ii", ta, tb))
    want = oracle.gemm(A, B)
    assert rel_err(host(C), want) <= TOL[dt]
    split_result = host(C).copy()
    if (dt, out) in EPI_KID:
        for relu in (1, 0):
            by_id(EPI_KID[(dt, out)], OpKind.GemmEpilogue, [X, W, Bv], [C], GPEL, struct.pack("<iii", ta, tb, relu))
            assert rel_err(host(C), oracle.gemm_epilogue(A, B, bias, False, False, bool(relu))) <= TOL[dt]
    # the unsplit kernel on the same operands: same product up to the order of the fp32 additions
    with gemm_tuning(splitk="0"):
        by_id(GEMM_KID[(dt, out)], OpKind.Gemm, [X, W], [C], GEMM, struct.pack("<ii", ta, tb))
    scale = float(np.abs(want).max())
    assert np.abs(host(C) - split_result).max() <= (2e-5 if out == "f32" else 1e-2) * scale
    assert _C.gemm_status() == 0


def test_gemm_split_over_k_with_relu_backward_mask_and_determinism(gpu):
    M, N, K = 96, 512, 4096
    A, B, bias, sa, sb = _operands(M, N, K, 0, 0, "bf16")
    Y = oracle.bf16_round(np.random.default_rng(5).standard_normal((M, N)).astype(np.float32))
    want = oracle.gemm_relu_bwd(A, B, Y)
    outs = []
    for force in ("4", "4", "0"):
        C = Tensor.zeros((M, N), "bf16")
        with gemm_tuning(splitk=force):
            by_id("gemm_relu_bwd_bf16_tcgen05_out_bf16_v0", OpKind.GemmReluBwd, [dev(sa, "bf16"), dev(sb, "bf16"), dev(Y, "bf16")],
                  [C], GEMM, struct.pack("<ii", 0, 0))
        assert rel_err(host(C), want) <= TOL["bf16"]
        assert np.array_equal(host(C) == 0, ~(Y > 0) | (host(C) == 0))
        outs.append(host(C))
    assert np.array_equal(outs[0], outs[1]), "parts are added in a fixed order"
    assert _C.gemm_status() == 0


# ------------------------------------------------------------------ last round of the paired kernel
def _sm_count():
    import ctypes as C
    import aicf_cuda
    sms = C.c_int(0)
    assert aicf_cuda.lib.aicf_b200_device_info(0, None, C.byref(sms), None) == 0
    return sms.value


def _gemm_workspace(kid, kind, ins, payload, schema):
    import aicf_cuda
    from aicf_cuda._C_ctypes import _blob, _build_descs
    descs = _build_descs(ins, "x")[0]
    blob, _keep = _blob(schema, payload)
    return aicf_cuda.lib.aicf_b200_query_workspace(kid.encode(), int(kind), descs, len(ins), blob)


def test_tuning_overrides_are_live_after_a_reload(gpu):
    """The launcher reads AICF_GEMM_* once per process; the tests' overrides only mean something because
    gemm_tuning() asks for a re-read. Observable through the workspace a shape asks for: a small batch against a long K
    is split over K (workspace for the parts) unless the split is switched off."""
    X, W = Tensor.empty((64, 4096), "bf16"), Tensor.empty((4096, 1024), "bf16")
    args = ("gemm_bf16_tcgen05_out_bf16_v0", OpKind.Gemm, [X, W], struct.pack("<ii", 0, 0), GEMM)
    assert _gemm_workspace(*args) > 0
    with gemm_tuning(splitk="0"):
        assert _gemm_workspace(*args) == 0
        with gemm_tuning(splitk="4", cta_group="1", tile_n="256"):
            assert _gemm_workspace(*args) == 4 * 64 * 1024 * 4
        assert _gemm_workspace(*args) == 0
    assert _gemm_workspace(*args) > 0


@pytest.mark.parametrize("rows_cut,cols_cut", [(0, 0), (60, 24)], ids=["whole_tiles", "ragged_edges"])
@pytest.mark.parametrize("K,tb", [(256, 1), (1088, 1), (1088, 0)])
def test_pair_kernel_tail_round_as_column_halves(gpu, K, tb, rows_cut, cols_cut):
    """One more round than the clusters can fill, with at most half of them busy: each left-over 256x256 tile is done as
    two 256x128 column halves on two clusters. Against fp64, and bit for bit against the same launch with the tail
    tiles left whole (every output element is still one accumulator over the same k order)."""
    clusters = _sm_count() // 2
    extra = max(1, min(6, clusters // 2))
    total = clusters + extra
    cols_t = 8 if total % 8 == 0 else 4 if total % 4 == 0 else 2 if total % 2 == 0 else 1
    M, N = total // cols_t * 256 - rows_cut, cols_t * 256 - cols_cut
    A, B, bias, sa, sb = _operands(M, N, K, 0, tb, "bf16", seed=11)
    X, W, Bv = dev(sa, "bf16"), dev(sb, "bf16"), dev(bias)
    kid, payload = "gemm_bias_relu_bf16_tcgen05_out_bf16_v0", struct.pack("<iii", 0, tb, 1)
    want = oracle.gemm_epilogue(A, B, bias, relu=True)
    outs = {}
    for mode, halves in [("halves", "1"), ("whole", "0")]:
        with gemm_tuning(cta_group="2", tail_halves=halves):
            C = dev(np.full((M, N), np.nan, np.float32), "bf16")  # an element nobody stores stays NaN
            by_id(kid, OpKind.GemmEpilogue, [X, W, Bv], [C], GPEL, payload)
            assert _C.gemm_status() == 0
            outs[mode] = host(C)
        assert rel_err(outs[mode], want) <= TOL["bf16"], mode
    assert np.array_equal(outs["halves"], outs["whole"])
    Y = oracle.bf16_round(np.random.default_rng(5).standard_normal((M, N)).astype(np.float32))
    with gemm_tuning(cta_group="2", tail_halves="1"):
        C32 = Tensor.zeros((M, N), "f32")
        by_id("gemm_bf16_tcgen05_out_f32_v0", OpKind.Gemm, [X, W], [C32], GEMM, struct.pack("<ii", 0, tb))
        Cm = Tensor.zeros((M, N), "bf16")
        by_id("gemm_relu_bwd_bf16_tcgen05_out_bf16_v0", OpKind.GemmReluBwd, [X, W, dev(Y, "bf16")], [Cm], GEMM, struct.pack("<ii", 0, tb))
        assert _C.gemm_status() == 0
    assert rel_err(host(C32), oracle.gemm(A, B)) <= 1e-4
    got = host(Cm)
    assert rel_err(got, oracle.gemm_relu_bwd(A, B, Y)) <= TOL["bf16"]
    assert not got[~(Y > 0)].any()
