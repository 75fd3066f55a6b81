"""Layer norm forward / backward through the binding against the fp64 oracle, and against the reference's own CUDA
kernels where the reference has them (f32, f16). Shapes cover the register path (one to eight packets per thread),
the multi-pass path (odd widths, unaligned views, rows past the register budget), single rows and single columns.
Tolerances: f32 1e-5 relative to the row scale; 16-bit outputs one rounding of the output type; parameter gradients
(f32 sums over M rows) 1e-5 of the sum of magnitudes."""
import struct

import numpy as np
import pytest

import oracle
from aicf_cuda import _C, Tensor
from aicf_cuda._C import OpKind
from util import by_id, dev, host, op_call, ref_by_id

pytestmark = pytest.mark.gpu

LNEP = 0x50454E4C
ROUND = {"f32": lambda a: np.asarray(a, np.float32), "f16": oracle.f16_round, "bf16": oracle.bf16_round}
EPS_OUT = {"f32": 1e-5, "f16": 1.0e-3, "bf16": 7.9e-3}  # relative rounding step of the output type (f32: the tolerance)

# (8,128), (64,256), (7,33) are the shapes of the reference's own layer-norm probe script
SHAPES = [(64, 1024), (33, 4096), (16, 8192), (8, 16384), (4, 20000), (5, 1001), (7, 3), (1, 256), (300, 64), (2, 40000),
          (129, 768), (8, 128), (64, 256), (7, 33)]


def make(M, N, dt, seed=0, offset=0.5):
    rng = np.random.default_rng(seed)
    x = ROUND[dt](rng.standard_normal((M, N)) * 2.0 + offset)
    dy = ROUND[dt](rng.standard_normal((M, N)))
    gamma = ROUND[dt](1.0 + 0.1 * rng.standard_normal(N))
    beta = ROUND[dt](0.1 * rng.standard_normal(N))
    return x, dy, gamma, beta


def fwd(dt, x, gamma=None, beta=None, eps=None, kid=None):
    M, N = x.shape
    ins = [dev(x, dt)] + ([dev(gamma, dt), dev(beta, dt)] if gamma is not None else [])
    outs = [Tensor.zeros((M, N), dt), Tensor.zeros((M,), "f32"), Tensor.zeros((M,), "f32")]
    schema, payload = (LNEP, struct.pack("<f", eps)) if eps is not None else (0, b"")
    if kid:
        by_id(kid, OpKind.LayerNormFwd, ins, outs, schema, payload)
    else:
        op_call(OpKind.LayerNormFwd, ins, outs, schema, payload)
    return [host(o) for o in outs]


def bwd(dt, x, dy, gamma, mean, rstd, kid=None):
    M, N = x.shape
    ins = [dev(x, dt), dev(dy, dt)] + ([dev(gamma, dt)] if gamma is not None else []) + [dev(mean), dev(rstd)]
    outs = [Tensor.zeros((M, N), dt)] + ([Tensor.zeros((N,), "f32"), Tensor.zeros((N,), "f32")] if gamma is not None else [])
    if kid:
        by_id(kid, OpKind.LayerNormBwd, ins, outs)
    else:
        op_call(OpKind.LayerNormBwd, ins, outs)
    return [host(o) for o in outs]


def close(got, want, dt, scale=None, what=""):
    want = np.asarray(want, np.float64)
    tol = EPS_OUT[dt] * (np.abs(want) + (scale if scale is not None else 1.0) * (1e-1 if dt == "f32" else 1.0)) + 1e-6
    err = np.abs(np.asarray(got, np.float64) - want)
    assert (err <= tol).all(), f"{what}: max err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}"


@pytest.mark.parametrize("M,N", SHAPES)
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_forward(gpu, M, N, dt, affine):
    x, _, gamma, beta = make(M, N, dt, seed=M + N)
    eps = np.float32(1e-5)
    y, mu, rs = fwd(dt, x, gamma if affine else None, beta if affine else None, eps=float(eps))
    wy, wmu, wrs = oracle.layernorm_fwd(x, gamma if affine else None, beta if affine else None, eps)
    np.testing.assert_allclose(mu, wmu, rtol=1e-5, atol=2e-6, err_msg="mean")
    np.testing.assert_allclose(rs, wrs, rtol=1e-5, err_msg="rstd")
    close(y, wy, dt, what="y")
    assert _C.wait_status() == 0


@pytest.mark.parametrize("M,N", SHAPES)
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_backward(gpu, M, N, dt, affine):
    x, dy, gamma, _ = make(M, N, dt, seed=M * 3 + N)
    _, mu, rs = oracle.layernorm_fwd(x, None, None, np.float32(1e-5))
    mu, rs = mu.astype(np.float32), rs.astype(np.float32)
    out = bwd(dt, x, dy, gamma if affine else None, mu, rs)
    wdx, wdg, wdb = oracle.layernorm_bwd(x, dy, gamma if affine else None, mu, rs)
    # dx = (N*g - s1 - xhat*s2) * rstd/N cancels: the error scales with |g| + |s1|/N + |xhat*s2|/N, i.e. O(rstd * |dy|)
    close(out[0], wdx, dt, scale=float(np.abs(wdx).max()), what="dx")
    if affine:
        xhat = (x.astype(np.float64) - mu[:, None]) * rs[:, None]
        np.testing.assert_array_less(np.abs(out[1] - wdg), 1e-5 * np.abs(dy * xhat).sum(axis=0) + 1e-6, err_msg="dgamma")
        np.testing.assert_array_less(np.abs(out[2] - wdb), 1e-5 * np.abs(dy).sum(axis=0) + 1e-6, err_msg="dbeta")
    assert _C.wait_status() == 0


def test_layernorm_defaults_ranks_and_rejections(gpu):
    x, dy, gamma, beta = make(12, 512, "f32", seed=9)
    # no attrs: eps = 1e-5; a custom eps changes rstd accordingly
    _, _, rs0 = fwd("f32", x)
    _, _, rs1 = fwd("f32", x, eps=0.5)
    var = x.astype(np.float64).var(axis=1)
    np.testing.assert_allclose(rs0, 1 / np.sqrt(var + 1e-5), rtol=1e-5)
    np.testing.assert_allclose(rs1, 1 / np.sqrt(var + 0.5), rtol=1e-5)
    # leading dimensions flatten: [3, 4, 512] is 12 rows
    X3 = dev(x.reshape(3, 4, 512))
    outs = [Tensor.zeros((3, 4, 512), "f32"), Tensor.zeros((12,), "f32"), Tensor.zeros((12,), "f32")]
    op_call(OpKind.LayerNormFwd, [X3, dev(gamma), dev(beta)], outs)
    np.testing.assert_allclose(host(outs[0]).reshape(12, 512), oracle.layernorm_fwd(x, gamma, beta, np.float32(1e-5))[0],
                               rtol=1e-5, atol=1e-5)
    # by-id dispatch picks the variant named, and a dtype it does not take is an error
    y16 = fwd("f16", oracle.f16_round(x), kid="layernorm_fwd_f16_v0")[0]
    assert np.isfinite(y16).all()
    with pytest.raises(RuntimeError):
        fwd("f32", x, kid="layernorm_fwd_f16_v0")
    # operand-count and shape errors
    M, N = x.shape
    good_out = lambda: [Tensor.zeros((M, N), "f32"), Tensor.zeros((M,), "f32"), Tensor.zeros((M,), "f32")]
    with pytest.raises(RuntimeError):
        op_call(OpKind.LayerNormFwd, [dev(x), dev(gamma)], good_out())                      # gamma without beta
    with pytest.raises(RuntimeError):
        op_call(OpKind.LayerNormFwd, [dev(x), dev(gamma[:-1]), dev(beta[:-1])], good_out())  # wrong parameter length
    with pytest.raises(RuntimeError):
        op_call(OpKind.LayerNormFwd, [dev(x)], [Tensor.zeros((M, N), "f32"), Tensor.zeros((M + 1,), "f32"), Tensor.zeros((M,), "f32")])
    with pytest.raises(RuntimeError):
        op_call(OpKind.LayerNormBwd, [dev(x), dev(dy), dev(gamma), dev(np.zeros(M, np.float32))], [Tensor.zeros((M, N), "f32")])


def test_layernorm_unaligned_views_take_the_multipass_path(gpu):
    M, N = 9, 1028
    x, dy, gamma, beta = make(M, N, "f32", seed=4)
    pad = lambda a: Tensor.from_numpy(np.concatenate([np.zeros(1, np.float32), a.ravel()]))
    bx, bdy = pad(x), pad(dy)
    vx = Tensor((M, N), "f32", ptr=bx.ptr + 4)
    vdy = Tensor((M, N), "f32", ptr=bdy.ptr + 4)
    outs = [Tensor.zeros((M, N), "f32"), Tensor.zeros((M,), "f32"), Tensor.zeros((M,), "f32")]
    op_call(OpKind.LayerNormFwd, [vx, dev(gamma), dev(beta)], outs)
    wy, wmu, wrs = oracle.layernorm_fwd(x, gamma, beta, np.float32(1e-5))
    np.testing.assert_allclose(host(outs[0]), wy, rtol=1e-5, atol=1e-5)
    mu, rs = wmu.astype(np.float32), wrs.astype(np.float32)
    bouts = [Tensor.zeros((M, N), "f32"), Tensor.zeros((N,), "f32"), Tensor.zeros((N,), "f32")]
    op_call(OpKind.LayerNormBwd, [vx, vdy, dev(gamma), dev(mu), dev(rs)], bouts)
    wdx, wdg, wdb = oracle.layernorm_bwd(x, dy, gamma, mu, rs)
    np.testing.assert_allclose(host(bouts[0]), wdx, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(host(bouts[1]), wdg, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(host(bouts[2]), wdb, rtol=1e-4, atol=1e-5)


def test_layernorm_backward_is_deterministic(gpu):
    x, dy, gamma, _ = make(2048, 1024, "f32", seed=5)
    _, mu, rs = oracle.layernorm_fwd(x, None, None, np.float32(1e-5))
    a = bwd("f32", x, dy, gamma, mu.astype(np.float32), rs.astype(np.float32))
    b = bwd("f32", x, dy, gamma, mu.astype(np.float32), rs.astype(np.float32))
    for u, v in zip(a, b):
        assert np.array_equal(u, v)


@pytest.mark.parametrize("M,N", [(64, 256), (37, 96), (128, 1024), (5, 1001), (8, 128), (7, 33), (16, 4096)])
@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_layernorm_vs_reference_kernels(ref_lib, M, N, dt):
    x, dy, gamma, beta = make(M, N, dt, seed=11)
    payload = struct.pack("<f", 1e-5)
    for affine in (True, False):
        ins = [dev(x, dt)] + ([dev(gamma, dt), dev(beta, dt)] if affine else [])
        specs = [((M, N), dt), ((M,), "f32"), ((M,), "f32")]
        ours = [Tensor.zeros(s, d) for s, d in specs]
        theirs = [Tensor.zeros(s, d) for s, d in specs]
        kid = f"layernorm_fwd_{dt}_v0"
        assert ref_by_id(ref_lib, kid, OpKind.LayerNormFwd, ins, theirs, LNEP, payload) == 0
        by_id(kid, OpKind.LayerNormFwd, ins, ours, LNEP, payload)
        np.testing.assert_allclose(host(ours[1]), host(theirs[1]), rtol=1e-5, atol=2e-6)
        np.testing.assert_allclose(host(ours[2]), host(theirs[2]), rtol=1e-5)
        close(host(ours[0]), host(theirs[0]), dt, what=f"y affine={affine}")
        # backward on the reference's own statistics
        bins = [dev(x, dt), dev(dy, dt)] + ([dev(gamma, dt)] if affine else []) + [theirs[1], theirs[2]]
        bspecs = [((M, N), dt)] + ([((N,), "f32"), ((N,), "f32")] if affine else [])
        bo = [Tensor.zeros(s, d) for s, d in bspecs]
        bt = [Tensor.zeros(s, d) for s, d in bspecs]
        kid = f"layernorm_bwd_{dt}_v0"
        assert ref_by_id(ref_lib, kid, OpKind.LayerNormBwd, bins, bt) == 0
        by_id(kid, OpKind.LayerNormBwd, bins, bo)
        close(host(bo[0]), host(bt[0]), dt, scale=float(np.abs(host(bt[0])).max()), what=f"dx affine={affine}")
        if affine:
            np.testing.assert_allclose(host(bo[1]), host(bt[1]), rtol=1e-4, atol=1e-4 * M ** 0.5)
            np.testing.assert_allclose(host(bo[2]), host(bt[2]), rtol=1e-4, atol=1e-4 * M ** 0.5)


@pytest.mark.parametrize("M,N,dt", [(4096, 1024, "f32"), (4096, 256, "bf16"), (2048, 4096, "bf16"), (512, 32000, "f32"),
                                    (8192, 96, "f16")])
def test_row_kernels_give_the_same_bits_every_time(gpu, M, N, dt):
    """The row kernels synchronise with two barriers per reduction over alternating shared-memory areas and take the
    row wait without a barrier; a hazard in that scheme would show up as run-to-run differences on many-row inputs."""
    x, dy, gamma, beta = make(M, N, dt, seed=21)
    X, DY, G, Bt = dev(x, dt), dev(dy, dt), dev(gamma, dt), dev(beta, dt)
    labels = dev(np.random.default_rng(3).integers(0, N, M).astype(np.int32))

    def once():
        out = {}
        y, mu, rs = Tensor.zeros((M, N), dt), Tensor.zeros((M,), "f32"), Tensor.zeros((M,), "f32")
        op_call(OpKind.LayerNormFwd, [X, G, Bt], [y, mu, rs])
        dx, dg, db = Tensor.zeros((M, N), dt), Tensor.zeros((N,), "f32"), Tensor.zeros((N,), "f32")
        op_call(OpKind.LayerNormBwd, [X, DY, G, mu, rs], [dx, dg, db])
        sm = Tensor.zeros((M, N), dt)
        op_call(OpKind.Softmax, [X], [sm])
        dz, loss, am = Tensor.zeros((M, N), dt), Tensor.zeros((M,), "f32"), Tensor.zeros((M,), "i32")
        op_call(OpKind.SoftmaxCE, [X, labels], [dz, loss, am])
        for k, t in dict(y=y, mu=mu, rs=rs, dx=dx, dg=dg, db=db, sm=sm, dz=dz, loss=loss, am=am).items():
            out[k] = t.numpy()
        return out

    first = once()
    for _ in range(5):
        again = once()
        for k in first:
            assert np.array_equal(first[k], again[k]), k
    assert _C.wait_status() == 0
